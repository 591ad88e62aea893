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
constexpr int SCAN_GROUPS = 16;      // row groups: thread (g, j) owns a run of rows of column j
constexpr int SCAN_MAX_ROWS = 16;    // rows per thread: dim up to 256
constexpr int SCAN_TOKENS = 4;       // tokens staged in shared memory a turn (one pair of barriers for all of them)
constexpr int SCAN_ITEMS = SCAN_TOKENS * SCAN_MAX_ROWS * SCAN_GROUPS / (SCAN_COLS * SCAN_GROUPS);   // staged items a thread

__device__ __forceinline__ float log_sigmoid(float z) {
    // log(1 / (1 + exp(-z))) without overflow on either side
    return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

// One kernel serves three uses.  A block walks tokens [t_lo, t_hi) of one sequence for one head and one
// tile of value columns:
//   whole run   (chunk = 0): from the slot's state, writing outputs, leaving the state in the slot;
//   chunk sums  (chunk > 0, sums != null, out == null): from zero over chunk blockIdx.x % max_chunks of the
//               sequence, leaving the chunk's own sum in ``sums`` and the product of its decays in ``decays``;
//   chunk outputs (chunk > 0, out != null): from the state at the chunk's start, which the carry kernel below
//               left in ``sums``, writing outputs.
// A long prompt is run as chunk sums, carry, chunk outputs: the chunks of a sequence in parallel, the same
// float32 recurrence within each.  Tokens are staged four at a time, and the next four are fetched while
// these are worked on.
// z <- sigmoid(z + bias)^(1 / tau), in place: the decays of every token and channel, once for all the blocks
// that walk them
__global__ void decay_kernel(float* __restrict__ z, int ldz, const float* __restrict__ z_bias, float inv_tau,
                             int width, size_t total) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / width;
    const int c = (int)(idx % width);
    float* p = z + t * ldz + c;
    *p = expf(log_sigmoid(*p + z_bias[c]) * inv_tau);
}

template <typename T>
__global__ void __launch_bounds__(SCAN_COLS * SCAN_GROUPS)
gated_linear_scan_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
                         const float* __restrict__ z, int ldz, float q_scale, float* __restrict__ state,
                         const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                         float* __restrict__ out, int ldo, int n_heads, int dim, int vdim,
                         int chunk, int max_chunks, float* __restrict__ sums, float* __restrict__ decays) {
    constexpr int NT = SCAN_COLS * SCAN_GROUPS;
    extern __shared__ __align__(16) float sm[];
    // rows per thread, a multiple of four: thread (g, j) owns rows g * rpt .. + rpt - 1 of column j, and reads
    // their decays, keys and queries four at a time; the arrays are padded with zeros up to 8 * rpt rows
    const int rpt = ((dim + SCAN_GROUPS - 1) / SCAN_GROUPS + 3) & ~3, dimp = rpt * SCAN_GROUPS;
    float* a_s = sm;                          // [SCAN_TOKENS][dimp] decays
    float* k_s = a_s + SCAN_TOKENS * dimp;    // [SCAN_TOKENS][dimp]
    float* q_s = k_s + SCAN_TOKENS * dimp;    // [SCAN_TOKENS][dimp]
    float* v_s = q_s + SCAN_TOKENS * dimp;    // [SCAN_TOKENS][SCAN_COLS]
    float* o_s = v_s + SCAN_TOKENS * SCAN_COLS;   // [SCAN_TOKENS][SCAN_GROUPS][SCAN_COLS]
    const int b = chunk > 0 ? blockIdx.x / max_chunks : blockIdx.x, c = chunk > 0 ? blockIdx.x % max_chunks : 0;
    const int h = blockIdx.y, j0 = blockIdx.z * SCAN_COLS;
    const int tid = threadIdx.x, j = tid % SCAN_COLS, g = tid / SCAN_COLS;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0) return;                                // padding row
    int t0 = cu_new[b], t1 = cu_new[b + 1];
    if (chunk > 0) {
        t0 += c * chunk;
        t1 = min(t1, t0 + chunk);
        if (t0 >= t1) return;
    }
    const bool col = j0 + j < vdim;
    const bool emit = out != nullptr;
    float* S = chunk > 0 ? sums + (((size_t)blockIdx.x * n_heads + h) * dim) * vdim
                         : state + ((size_t)slot * n_heads + h) * dim * vdim;
    float s_reg[SCAN_MAX_ROWS];
#pragma unroll
    for (int r = 0; r < SCAN_MAX_ROWS; ++r) {
        const int i = g * rpt + r;
        s_reg[r] = (col && r < rpt && i < dim && (chunk == 0 || emit)) ? S[(size_t)i * vdim + j0 + j] : 0.f;
    }
    for (int e = tid; e < 3 * SCAN_TOKENS * dimp; e += NT) sm[e] = 0.f;      // the padding stays zero
    // a turn stages SCAN_TOKENS tokens: item (token, channel) n * NT + tid of the turn is this thread's
    float zz[SCAN_ITEMS], kk[SCAN_ITEMS], qq[SCAN_ITEMS], vv = 0.f, a_prod = 1.f;
    int item_tt[SCAN_ITEMS], item_i[SCAN_ITEMS];         // the same in every turn: divided once
#pragma unroll
    for (int n = 0; n < SCAN_ITEMS; ++n) {
        const int item = n * NT + tid;
        item_tt[n] = item < SCAN_TOKENS * dim ? item / dim : SCAN_TOKENS;
        item_i[n] = item % dim;
    }
    auto fetch = [&](int t) {
        const int n_tok = min(SCAN_TOKENS, t1 - t);
#pragma unroll
        for (int n = 0; n < SCAN_ITEMS; ++n) {
            const int tt = item_tt[n], i = item_i[n];
            if (tt < n_tok) {
                const T* row = proj + (size_t)(t + tt) * ld;
                zz[n] = z[(size_t)(t + tt) * ldz + h * dim + i];
                kk[n] = ssb_to_float(row[k_off + h * dim + i]);
                qq[n] = ssb_to_float(row[q_off + h * dim + i]);
            }
        }
        if (tid < SCAN_TOKENS * SCAN_COLS) {
            const int tt = tid / SCAN_COLS, jj = tid % SCAN_COLS;
            vv = (tt < n_tok && j0 + jj < vdim) ? ssb_to_float(proj[(size_t)(t + tt) * ld + v_off + h * vdim + j0 + jj]) : 0.f;
        }
    };
    fetch(t0);
    __syncthreads();
    for (int t = t0; t < t1; t += SCAN_TOKENS) {
        const int n_tok = min(SCAN_TOKENS, t1 - t);
#pragma unroll
        for (int n = 0; n < SCAN_ITEMS; ++n) {
            const int tt = item_tt[n], i = item_i[n];
            if (tt < n_tok) {
                a_s[tt * dimp + i] = zz[n];
                k_s[tt * dimp + i] = kk[n];
                q_s[tt * dimp + i] = qq[n] * q_scale;
            }
        }
        if (tid < SCAN_TOKENS * SCAN_COLS) v_s[tid] = vv;
        __syncthreads();
        if (t + SCAN_TOKENS < t1) fetch(t + SCAN_TOKENS);
        if (decays != nullptr && tid < dim)
            for (int tt = 0; tt < n_tok; ++tt) a_prod *= a_s[tt * dimp + tid];
        for (int tt = 0; tt < n_tok; ++tt) {
            const float v = v_s[tt * SCAN_COLS + j];
            const float4* a4 = reinterpret_cast<const float4*>(a_s + tt * dimp + g * rpt);
            const float4* k4 = reinterpret_cast<const float4*>(k_s + tt * dimp + g * rpt);
            const float4* q4 = reinterpret_cast<const float4*>(q_s + tt * dimp + g * rpt);
            float o = 0.f;
#pragma unroll
            for (int r = 0; r < SCAN_MAX_ROWS; r += 4)
                if (r < rpt) {
                    const float4 a = a4[r >> 2], k = k4[r >> 2], q = q4[r >> 2];
                    s_reg[r] = fmaf(a.x, s_reg[r], k.x * v);          o = fmaf(s_reg[r], q.x, o);
                    s_reg[r + 1] = fmaf(a.y, s_reg[r + 1], k.y * v);  o = fmaf(s_reg[r + 1], q.y, o);
                    s_reg[r + 2] = fmaf(a.z, s_reg[r + 2], k.z * v);  o = fmaf(s_reg[r + 2], q.z, o);
                    s_reg[r + 3] = fmaf(a.w, s_reg[r + 3], k.w * v);  o = fmaf(s_reg[r + 3], q.w, o);
                }
            if (emit) o_s[(tt * SCAN_GROUPS + g) * SCAN_COLS + j] = o;
        }
        __syncthreads();
        if (emit && tid < n_tok * SCAN_COLS) {
            const int tt = tid / SCAN_COLS, jj = tid % SCAN_COLS;
            if (j0 + jj < vdim) {
                float sum = 0.f;
#pragma unroll
                for (int gg = 0; gg < SCAN_GROUPS; ++gg) sum += o_s[(tt * SCAN_GROUPS + gg) * SCAN_COLS + jj];
                out[(size_t)(t + tt) * ldo + h * vdim + j0 + jj] = sum;
            }
        }
    }
    if (chunk > 0 && emit) return;                       // the state was carried by the carry kernel
#pragma unroll
    for (int r = 0; r < SCAN_MAX_ROWS; ++r) {
        const int i = g * rpt + r;
        if (col && r < rpt && i < dim) S[(size_t)i * vdim + j0 + j] = s_reg[r];
    }
    if (chunk > 0 && blockIdx.z == 0 && tid < dim) decays[((size_t)blockIdx.x * n_heads + h) * dim + tid] = a_prod;
}

// Carries the state across a sequence's chunks: with S the state before chunk c, chunk c's place in
// ``sums`` gets S (what the chunk starts from) and S <- decays[c] * S + sums[c]; the last S is the
// sequence's state.  One thread per state element, chunks in order.
__global__ void __launch_bounds__(256)
gated_linear_carry_kernel(float* __restrict__ state, float* __restrict__ sums, const float* __restrict__ decays,
                          const int* __restrict__ cu_new, const int* __restrict__ seq_slot, int n_heads, int dim,
                          int vdim, int chunk, int max_chunks) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int b = blockIdx.y, slot = seq_slot[b];
    if (slot < 0) return;
    const size_t per = (size_t)n_heads * dim * vdim;
    const size_t e = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (e >= per) return;
    const size_t hi = e / vdim;                          // head * dim + channel
    const int n_chunks = (cu_new[b + 1] - cu_new[b] + chunk - 1) / chunk;
    float cur = state[(size_t)slot * per + e];
    float* sp = sums + (size_t)b * max_chunks * per + e;
    const float* dp = decays + (size_t)b * max_chunks * n_heads * dim + hi;
    float loc = n_chunks > 0 ? sp[0] : 0.f, a = n_chunks > 0 ? dp[0] : 0.f;
    for (int c = 0; c < n_chunks; ++c) {
        float loc_n = 0.f, a_n = 0.f;
        if (c + 1 < n_chunks) {
            loc_n = sp[(size_t)(c + 1) * per];
            a_n = dp[(size_t)(c + 1) * n_heads * dim];
        }
        sp[(size_t)c * per] = cur;
        cur = fmaf(a, cur, loc);
        loc = loc_n;
        a = a_n;
    }
    state[(size_t)slot * per + e] = cur;
}

// proj [T, ld] holds q, k (n_heads x dim each) and v (n_heads x vdim) from the given columns;
// z [T, ldz] float32 is the decay's pre-activation without its bias z_bias [n_heads x dim], and is overwritten
// with the decays;
// state [slots, n_heads, dim, vdim] float32; out [T, ldo] float32 gets o (n_heads x vdim).
// chunk > 0: sequences are run in chunks of that many tokens, in parallel, through ``sums``
// (n_seqs x max_chunks x n_heads x dim x vdim floats) and ``decays`` (n_seqs x max_chunks x n_heads x dim);
// max_chunks = ceil(longest run of new tokens / chunk).
SSB_API int ssb_gated_linear_scan(const void* proj, int ld, int dtype, int q_off, int k_off, int v_off,
                                  float* z, int ldz, const float* z_bias, float tau, float q_scale,
                                  float* state, const int* cu_new, const int* seq_slot, float* out, int ldo,
                                  int n_seqs, int n_tokens, int n_heads, int dim, int vdim, int chunk, int max_chunks,
                                  float* sums, float* decays, int pdl, cudaStream_t stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (dim <= 0 || dim > SCAN_MAX_ROWS * SCAN_GROUPS || vdim <= 0 || !(tau > 0.f)) return SSB_ERR_BAD_SIZE;
    if (chunk < 0 || (chunk > 0 && (max_chunks <= 0 || sums == nullptr || decays == nullptr))) return SSB_ERR_BAD_SIZE;
    const long long items = chunk > 0 ? (long long)n_seqs * max_chunks : n_seqs;
    if (items > 0x7fffffffll) return SSB_ERR_BAD_SIZE;
    const dim3 grid((unsigned)items, n_heads, (vdim + SCAN_COLS - 1) / SCAN_COLS);
    if (grid.y > 65535 || grid.z > 65535 || n_seqs > 65535) return SSB_ERR_BAD_SIZE;
    const int rpt = ((dim + SCAN_GROUPS - 1) / SCAN_GROUPS + 3) & ~3;
    const size_t smem = (size_t)SCAN_TOKENS * (3 * rpt * SCAN_GROUPS + SCAN_COLS + SCAN_COLS * SCAN_GROUPS) * sizeof(float);
    int rc = 0;
    {
        const size_t total = (size_t)n_tokens * n_heads * dim;
        rc = ssb_launch(decay_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, pdl != 0, z, ldz, z_bias,
                        1.0f / tau, n_heads * dim, total);
        if (!rc) rc = ssb_launch_status();
        if (rc) return rc;
    }
#define SSB_SCAN(T, OUT) \
    rc = ssb_launch(gated_linear_scan_kernel<T>, grid, dim3(SCAN_COLS * SCAN_GROUPS), smem, stream, pdl != 0, \
                    (const T*)proj, ld, q_off, k_off, v_off, (const float*)z, ldz, q_scale, state, cu_new, seq_slot, \
                    OUT, ldo, n_heads, dim, vdim, chunk, max_chunks, sums, decays)
#define SSB_SCAN_BOTH(OUT) do { \
        if (dtype == SSB_F32) SSB_SCAN(float, OUT); \
        else if (dtype == SSB_BF16) SSB_SCAN(bf16, OUT); \
        else return SSB_ERR_BAD_DTYPE; \
        if (!rc) rc = ssb_launch_status(); \
        if (rc) return rc; \
    } while (0)
    if (chunk == 0) {
        SSB_SCAN_BOTH(out);
        return 0;
    }
    SSB_SCAN_BOTH((float*)nullptr);
    const size_t per = (size_t)n_heads * dim * vdim;
    rc = ssb_launch(gated_linear_carry_kernel, dim3((unsigned)((per + 255) / 256), n_seqs), dim3(256), 0, stream, pdl != 0,
                    state, sums, (const float*)decays, cu_new, seq_slot, n_heads, dim, vdim, chunk, max_chunks);
    if (!rc) rc = ssb_launch_status();
    if (rc) return rc;
    SSB_SCAN_BOTH(out);
#undef SSB_SCAN_BOTH
#undef SSB_SCAN
    return 0;
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
