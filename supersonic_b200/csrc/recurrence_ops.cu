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
#include <type_traits>

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
// y[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * w * act(gate[t, h, :]): a head's
// output normalised over its own width, weighted (one weight vector for all heads, or w_stride = vdim:
// one per head), then gated; act is silu (gate_kind 0), sigmoid (1), or the gate as it is (2: the
// caller has applied its activation already)
// ---------------------------------------------------------------------------------------
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, int ldo, const TW* __restrict__ w, int w_stride, float eps,
                      const T* __restrict__ gate, int ldg, int gate_kind, T* __restrict__ y, int ldy, int vdim, int n_heads) {
    // a warp per (token, head): its lanes walk the head's columns and meet in shuffles
    const int t = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    if (h >= n_heads) return;
    const float* src = o + (size_t)t * ldo + (size_t)h * vdim;
    float part = 0.f;
    for (int c = lane; c < vdim; c += 32) part = fmaf(src[c], src[c], part);
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
    const float inv = 1.0f / sqrtf(part / (float)vdim + eps);
    const T* gr = gate + (size_t)t * ldg + (size_t)h * vdim;
    const TW* wr = w + (size_t)h * w_stride;
    T* dst = y + (size_t)t * ldy + (size_t)h * vdim;
    for (int c = lane; c < vdim; c += 32) {
        const float gv = ssb_to_float(gr[c]);
        const float sg = 1.0f / (1.0f + expf(-gv));
        const float ga = gate_kind == 0 ? gv * sg : gate_kind == 1 ? sg : gv;
        dst[c] = ssb_from_float<T>(src[c] * inv * ssb_to_float(wr[c]) * ga);
    }
}

SSB_API int ssb_head_norm_gate(const float* o, int ldo, const void* w, int w_dtype, int w_stride, float eps,
                               const void* gate, int ldg, int gate_kind, void* y, int ldy, int dtype, int n_tokens,
                               int n_heads, int vdim, int pdl, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (vdim <= 0 || n_heads <= 0 || n_heads > 65535 || gate_kind < 0 || gate_kind > 2) return SSB_ERR_BAD_SIZE;
    const dim3 grid(n_tokens, (n_heads + 3) / 4);
    int rc = 0;
#define SSB_HNG(T, TW) \
    rc = ssb_launch(head_norm_gate_kernel<T, TW>, grid, dim3(128), 0, stream, pdl != 0, o, ldo, (const TW*)w, w_stride, eps, \
                    (const T*)gate, ldg, gate_kind, (T*)y, ldy, vdim, n_heads)
    if (dtype == SSB_F32 && w_dtype == SSB_F32) SSB_HNG(float, float);
    else if (dtype == SSB_BF16 && w_dtype == SSB_BF16) SSB_HNG(bf16, bf16);
    else if (dtype == SSB_BF16 && w_dtype == SSB_F32) SSB_HNG(bf16, float);
    else if (dtype == SSB_F32 && w_dtype == SSB_BF16) SSB_HNG(float, bf16);
    else return SSB_ERR_BAD_DTYPE;
#undef SSB_HNG
    return rc ? rc : ssb_launch_status();
}

// =======================================================================================
// Two more recurrences over a matrix state S [dim, vdim] per head, and one over a vector state.
//
// Delta rule with decay and removal (DELTA): with a unit key u and a removal rate a per key channel,
//     S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,    o_t = S_t^T r_t
// (both the decayed and the removed part read the old state).
// Decay with a bonus for the token at hand (!DELTA):
//     o_t = (S_(t-1) + diag(b) k_t v_t^T)^T r_t,    S_t = diag(w_t) S_(t-1) + k_t v_t^T
// What enters besides r, k and v (the decays w, u, a * u) is float32 and made by the prepare kernel below.
// =======================================================================================
constexpr int MS_LANES = 8;          // lanes that share a value column: each owns a run of its rows
constexpr int MS_COLS = 16;          // value columns a block of 128 threads owns
constexpr int MS_TOKENS = 4;         // tokens staged per pair of barriers
constexpr int MS_THREADS = MS_LANES * MS_COLS;

// Decays in place and, for the delta rule, unit keys and removal vectors.  One warp per (token, head).
//   decay_kind 0: z <- exp(-exp(z + z_bias));  1: z <- exp(-decay_scale * sigmoid(z + z_bias));
//   log_decay: z gets the decay's logarithm instead (the float32 path's scan takes the exponential in double)
//   with_unit: unit[t] = [u | a * u], u = k / sqrt(sum(k^2) + unit_eps), a = sigmoid(a_pre + a_bias)
template <typename T>
__global__ void __launch_bounds__(128)
state_scan_prepare_kernel(float* __restrict__ z, int ldz, const float* __restrict__ z_bias, int decay_kind,
                          int log_decay, float decay_scale, const T* __restrict__ proj, int ld, int k_off, int a_off,
                          const float* __restrict__ a_bias, float unit_eps, float* __restrict__ unit, int ldu,
                          int n_heads, int dim) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const size_t t = blockIdx.x;
    const int h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;     // a warp per (token, head)
    if (h >= n_heads) return;
    float* zr = z + t * ldz + (size_t)h * dim;
    for (int i = lane; i < dim; i += 32) {
        const float v = zr[i] + z_bias[h * dim + i];
        const float lw = decay_kind == 0 ? -expf(v) : -decay_scale / (1.0f + expf(-v));
        zr[i] = log_decay ? lw : expf(lw);
    }
    if (unit == nullptr) return;
    const T* kr = proj + t * ld + k_off + (size_t)h * dim;
    const T* ar = proj + t * ld + a_off + (size_t)h * dim;
    float part = 0.f;
    for (int i = lane; i < dim; i += 32) {
        const float k = ssb_to_float(kr[i]);
        part = fmaf(k, k, part);
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
    const float inv = 1.0f / sqrtf(part + unit_eps);
    float* ur = unit + t * ldu + (size_t)h * dim;
    float* aur = ur + (size_t)n_heads * dim;
    for (int i = lane; i < dim; i += 32) {
        const float u = ssb_to_float(kr[i]) * inv;
        const float a = 1.0f / (1.0f + expf(-(ssb_to_float(ar[i]) + a_bias[h * dim + i])));
        ur[i] = u;
        aur[i] = a * u;
    }
}

SSB_API int ssb_state_scan_prepare(float* z, int ldz, const float* z_bias, int decay_kind, int log_decay, float decay_scale,
                                   const void* proj, int ld, int dtype, int k_off, int a_off, const float* a_bias,
                                   float unit_eps, float* unit, int ldu, int n_tokens, int n_heads, int dim, int pdl,
                                   cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_heads <= 0 || n_heads > 65535 || dim <= 0 || decay_kind < 0 || decay_kind > 1) return SSB_ERR_BAD_SIZE;
    const dim3 grid(n_tokens, (n_heads + 3) / 4);
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(state_scan_prepare_kernel<float>, grid, dim3(128), 0, stream, pdl != 0, z, ldz, z_bias, decay_kind,
                        log_decay, decay_scale, (const float*)proj, ld, k_off, a_off, a_bias, unit_eps, unit, ldu, n_heads, dim);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(state_scan_prepare_kernel<bf16>, grid, dim3(128), 0, stream, pdl != 0, z, ldz, z_bias, decay_kind,
                        log_decay, decay_scale, (const bf16*)proj, ld, k_off, a_off, a_bias, unit_eps, unit, ldu, n_heads, dim);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}

// A block walks the new tokens of one sequence for one head and 16 value columns.  Eight lanes share a
// column: lane s owns rows s * RPL .. s * RPL + RPL - 1 of it in registers, and the sums over rows that a
// token needs (u^T S before the update, S^T r after it) are three shuffle steps.  The vectors of four
// tokens are staged in shared memory per pair of barriers while the next four are on their way.
template <typename T, int RPL, bool DELTA>
__global__ void __launch_bounds__(MS_THREADS)
matrix_state_scan_kernel(const T* __restrict__ proj, int ld, int r_off, int k_off, int v_off,
                         const float* __restrict__ decay, int ldd, const float* __restrict__ unit, int ldu,
                         const float* __restrict__ bonus, float* __restrict__ state, const int* __restrict__ cu_new,
                         const int* __restrict__ seq_slot, float* __restrict__ out, int ldo, int n_heads, int dim,
                         int vdim) {
    constexpr int DIMP = MS_LANES * RPL;                 // padded rows
    constexpr int NV = DELTA ? 5 : 3;                    // staged vectors per token: w, k, r (, u, a * u)
    constexpr int ITEMS = (MS_TOKENS * NV * DIMP + MS_THREADS - 1) / MS_THREADS;
    __shared__ __align__(16) float vec[NV][MS_TOKENS][DIMP];
    __shared__ float v_s[MS_TOKENS][MS_COLS];
    const int b = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * MS_COLS;
    const int tid = threadIdx.x, sub = tid % MS_LANES, cj = tid / MS_LANES;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t0 = cu_new[b], t1 = cu_new[b + 1];
    if (t0 >= t1) return;
    const bool col = j0 + cj < vdim;
    float* S = state + ((size_t)slot * n_heads + h) * dim * vdim;
    // the float32 path (T = float) carries the state of a step's tokens in double and is given the decays'
    // logarithms, of which it takes the exponential in double: a decay within 1e-3 of one, rounded to float32,
    // is off by 1e-4 of its logarithm, the same way at every token if its input hardly changes
    constexpr bool PRECISE = std::is_same<T, float>::value;
    using A = typename std::conditional<PRECISE, double, float>::type;
    A s_reg[RPL];
    float b_reg[RPL];
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = sub * RPL + r;
        s_reg[r] = (col && i < dim) ? S[(size_t)(j0 + cj) * dim + i] : 0.f;
        b_reg[r] = (!DELTA && bonus != nullptr && i < dim) ? bonus[h * dim + i] : 0.f;
    }
    for (int e = tid; e < NV * MS_TOKENS * DIMP; e += MS_THREADS) (&vec[0][0][0])[e] = 0.f;   // the padding stays zero
    // item n * MS_THREADS + tid of a turn is (vector, token, channel); the same in every turn
    float val[ITEMS], vv = 0.f;
    int item_v[ITEMS], item_tt[ITEMS], item_i[ITEMS];
#pragma unroll
    for (int n = 0; n < ITEMS; ++n) {
        const int item = n * MS_THREADS + tid;
        const int per = MS_TOKENS * dim;
        item_v[n] = item < NV * per ? item / per : NV;
        item_tt[n] = (item % per) / dim;
        item_i[n] = item % dim;
    }
    auto fetch = [&](int t) {
        const int n_tok = min(MS_TOKENS, t1 - t);
#pragma unroll
        for (int n = 0; n < ITEMS; ++n) {
            const int v = item_v[n], tt = item_tt[n], i = item_i[n];
            if (v < NV && tt < n_tok) {
                const size_t row = (size_t)(t + tt);
                const int c = h * dim + i;
                val[n] = v == 0 ? decay[row * ldd + c]
                       : v == 1 ? ssb_to_float(proj[row * ld + k_off + c])
                       : v == 2 ? ssb_to_float(proj[row * ld + r_off + c])
                       : v == 3 ? unit[row * ldu + c]
                                : unit[row * ldu + n_heads * dim + c];
            }
        }
        if (tid < MS_TOKENS * MS_COLS) {
            const int tt = tid / MS_COLS, jj = tid % MS_COLS;
            vv = (tt < n_tok && j0 + jj < vdim) ? ssb_to_float(proj[(size_t)(t + tt) * ld + v_off + h * vdim + j0 + jj]) : 0.f;
        }
    };
    fetch(t0);
    __syncthreads();
    for (int t = t0; t < t1; t += MS_TOKENS) {
        const int n_tok = min(MS_TOKENS, t1 - t);
#pragma unroll
        for (int n = 0; n < ITEMS; ++n)
            if (item_v[n] < NV && item_tt[n] < n_tok) vec[item_v[n]][item_tt[n]][item_i[n]] = val[n];
        if (tid < MS_TOKENS * MS_COLS) v_s[tid / MS_COLS][tid % MS_COLS] = vv;
        __syncthreads();
        if (t + MS_TOKENS < t1) fetch(t + MS_TOKENS);
        for (int tt = 0; tt < n_tok; ++tt) {
            const float v = v_s[tt][cj];
            const float4* w4 = reinterpret_cast<const float4*>(&vec[0][tt][sub * RPL]);
            const float4* k4 = reinterpret_cast<const float4*>(&vec[1][tt][sub * RPL]);
            const float4* r4 = reinterpret_cast<const float4*>(&vec[2][tt][sub * RPL]);
            A o = 0;
            const float* wv = &vec[0][tt][sub * RPL];
            const float* kvv = &vec[1][tt][sub * RPL];
            const float* rv = &vec[2][tt][sub * RPL];
            if (DELTA) {
                const float* uv = &vec[NV - 2][tt][sub * RPL];
                const float* auv = &vec[NV - 1][tt][sub * RPL];
                A seen = 0;
#pragma unroll
                for (int r = 0; r < RPL; r += 4) {
                    const float4 u = *reinterpret_cast<const float4*>(uv + r);
                    seen += (A)u.x * s_reg[r] + (A)u.y * s_reg[r + 1] + (A)u.z * s_reg[r + 2] + (A)u.w * s_reg[r + 3];
                }
                seen += __shfl_xor_sync(0xffffffffu, seen, 1);
                seen += __shfl_xor_sync(0xffffffffu, seen, 2);
                seen += __shfl_xor_sync(0xffffffffu, seen, 4);
#pragma unroll
                for (int r = 0; r < RPL; r += 4) {
                    const float4 w = *reinterpret_cast<const float4*>(wv + r), k = *reinterpret_cast<const float4*>(kvv + r);
                    const float4 q = *reinterpret_cast<const float4*>(rv + r), au = *reinterpret_cast<const float4*>(auv + r);
                    const float ww[4] = {w.x, w.y, w.z, w.w}, kk[4] = {k.x, k.y, k.z, k.w};
                    const float qq[4] = {q.x, q.y, q.z, q.w}, aa[4] = {au.x, au.y, au.z, au.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const A dec = PRECISE ? (A)exp((double)ww[e]) : (A)ww[e];
                        s_reg[r + e] = dec * s_reg[r + e] + ((A)kk[e] * (A)v - (A)aa[e] * seen);
                        o += s_reg[r + e] * (A)qq[e];
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < RPL; r += 4) {
                    const float4 w = *reinterpret_cast<const float4*>(wv + r), k = *reinterpret_cast<const float4*>(kvv + r);
                    const float4 q = *reinterpret_cast<const float4*>(rv + r);
                    const float ww[4] = {w.x, w.y, w.z, w.w}, kk[4] = {k.x, k.y, k.z, k.w}, qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const A dec = PRECISE ? (A)exp((double)ww[e]) : (A)ww[e];
                        const A kv = (A)kk[e] * (A)v;
                        o += ((A)b_reg[r + e] * kv + s_reg[r + e]) * (A)qq[e];
                        s_reg[r + e] = dec * s_reg[r + e] + kv;
                    }
                }
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);
            if (sub == 0 && col) out[(size_t)(t + tt) * ldo + h * vdim + j0 + cj] = (float)o;
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = sub * RPL + r;
        if (col && i < dim) S[(size_t)(j0 + cj) * dim + i] = (float)s_reg[r];
    }
}

// The same walk for bfloat16 projections whose rows can be fetched in 16-byte pieces: the vectors of four tokens
// a stage go from global to shared memory by cp.async in the types they are stored in (decays and unit keys
// float32, r, k and v bfloat16), four stages deep, so that the loads of the next twelve tokens are in flight
// while four are worked on, with one barrier per four tokens.  (With the vectors staged through registers the
// walk waited on global memory at every turn: four warps an SM hide nothing.)  LANES lanes share a column: sixteen
// where a head has 64 key channels or more (a lane's share of a token is then half as many instructions, and the
// walk is bound by the instructions one warp issues a token), eight otherwise.
template <int LANES, int RPL, bool DELTA>
__global__ void __launch_bounds__(MS_THREADS)
matrix_state_scan_async_kernel(const bf16* __restrict__ proj, int ld, int r_off, int k_off, int v_off,
                               const float* __restrict__ decay, int ldd, const float* __restrict__ unit, int ldu,
                               const float* __restrict__ bonus, float* __restrict__ state,
                               const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                               float* __restrict__ out, int ldo, int n_heads, int dim, int vdim) {
    constexpr int COLS = MS_THREADS / LANES;              // value columns a block owns: 16 with eight lanes a column, 8 with sixteen
    constexpr int DIMP = LANES * RPL, STAGES = 4, TOK = MS_TOKENS;
    constexpr int NF = DELTA ? 3 : 1;                    // float32 vectors a token: w (, u, a * u)
    constexpr int F_BYTES = NF * TOK * DIMP * 4, KR_BYTES = 2 * TOK * DIMP * 2, V_BYTES = TOK * COLS * 2;
    constexpr int STAGE_BYTES = F_BYTES + KR_BYTES + V_BYTES;
    extern __shared__ __align__(16) unsigned char ms_smem[];
    const int b = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * COLS;
    const int tid = threadIdx.x, sub = tid % LANES, cj = tid / LANES;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t0 = cu_new[b], t1 = cu_new[b + 1];
    if (t0 >= t1) return;
    const bool col = j0 + cj < vdim;
    float* S = state + ((size_t)slot * n_heads + h) * dim * vdim;
    float s_reg[RPL], b_reg[RPL];
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = sub * RPL + r;
        s_reg[r] = (col && i < dim) ? S[(size_t)(j0 + cj) * dim + i] : 0.f;
        b_reg[r] = (!DELTA && bonus != nullptr && i < dim) ? bonus[h * dim + i] : 0.f;
    }
    if (dim < DIMP || j0 + COLS > vdim) {             // rows past dim and columns past vdim are never copied: they stay zero
        for (int e = tid; e < STAGES * STAGE_BYTES / 4; e += MS_THREADS) reinterpret_cast<uint32_t*>(ms_smem)[e] = 0u;
        __syncthreads();
    }
    // the 16-byte pieces of a stage are the same in every stage but for the token they start from: each thread
    // works out its pieces once (where in a row, which array, where in the stage) and only adds the row offset
    constexpr int VP = COLS / 8;                           // 16-byte pieces of a token's value columns
    constexpr int NCH = (TOK * (NF * (DIMP / 4) + 2 * (DIMP / 8) + VP) + MS_THREADS - 1) / MS_THREADS;
    const int cf = dim / 4, cb = dim / 8, per_tok = NF * cf + 2 * cb + VP;
    const unsigned char* c_src[NCH];
    long long c_step[NCH];                               // bytes from a row to the next in the piece's array
    int c_dst[NCH], c_tt[NCH];                           // c_tt = TOK: no piece
#pragma unroll
    for (int n = 0; n < NCH; ++n) {
        const int c = n * MS_THREADS + tid;
        c_tt[n] = TOK;
        c_src[n] = nullptr;
        c_step[n] = 0;
        c_dst[n] = 0;
        if (c >= TOK * per_tok) continue;
        const int tt = c / per_tok;
        int e = c % per_tok;
        if (e < NF * cf) {
            const int vid = e / cf, ch = e % cf;
            const float* base = vid == 0 ? decay : unit + (size_t)(vid - 1) * n_heads * dim;
            c_step[n] = (long long)(vid == 0 ? ldd : ldu) * 4;
            c_src[n] = reinterpret_cast<const unsigned char*>(base + h * dim + ch * 4) + (size_t)(t0 + tt) * c_step[n];
            c_dst[n] = ((vid * TOK + tt) * DIMP + ch * 4) * 4;
        } else if ((e -= NF * cf) < 2 * cb) {
            const int which = e / cb, ch = e % cb;       // 0: k, 1: r
            c_step[n] = (long long)ld * 2;
            c_src[n] = reinterpret_cast<const unsigned char*>(proj + (which ? r_off : k_off) + h * dim + ch * 8) +
                       (size_t)(t0 + tt) * c_step[n];
            c_dst[n] = F_BYTES + ((which * TOK + tt) * DIMP + ch * 8) * 2;
        } else {
            e -= 2 * cb;
            if (j0 + e * 8 >= vdim) continue;
            c_step[n] = (long long)ld * 2;
            c_src[n] = reinterpret_cast<const unsigned char*>(proj + v_off + h * vdim + j0 + e * 8) + (size_t)(t0 + tt) * c_step[n];
            c_dst[n] = F_BYTES + KR_BYTES + (tt * COLS + e * 8) * 2;
        }
        c_tt[n] = tt;
    }
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(ms_smem);
    auto issue = [&](int t, int stage) {
        const int n_tok = max(0, min(TOK, t1 - t));
        const long long rows = t - t0;
#pragma unroll
        for (int n = 0; n < NCH; ++n)
            if (c_tt[n] < n_tok)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_base + stage * STAGE_BYTES + c_dst[n]),
                             "l"(c_src[n] + rows * c_step[n]) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) issue(t0 + st * TOK, st);
    int it = 0;
    for (int t = t0; t < t1; t += TOK, ++it) {
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
        __syncthreads();                                 // this stage has landed; everyone is done with the one before
        issue(t + (STAGES - 1) * TOK, (it + STAGES - 1) % STAGES);
        const unsigned char* base = ms_smem + (it % STAGES) * STAGE_BYTES;
        const float* fv = reinterpret_cast<const float*>(base);
        const bf16* kr = reinterpret_cast<const bf16*>(base + F_BYTES);
        const bf16* vs = reinterpret_cast<const bf16*>(base + F_BYTES + KR_BYTES);
        const int n_tok = min(TOK, t1 - t);
        // the four tokens of a stage unrolled: the loads and conversions of a token overlap the chain of the one
        // before, and the sums over a column's lanes for the outputs are taken for all four at the end
        float o_part[TOK];
#pragma unroll
        for (int tt = 0; tt < TOK; ++tt) {
            o_part[tt] = 0.f;
            if (tt >= n_tok) continue;                   // only a sequence's last stage is short
            const float v = __bfloat162float(vs[tt * COLS + cj]);
            const float* wv = fv + tt * DIMP + sub * RPL;
            const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(kr + tt * DIMP + sub * RPL);
            const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(kr + (TOK + tt) * DIMP + sub * RPL);
            float o0 = 0.f, o1 = 0.f;
            if (DELTA) {
                const float* uv = fv + (TOK + tt) * DIMP + sub * RPL;
                const float* auv = fv + (2 * TOK + tt) * DIMP + sub * RPL;
                float seen0 = 0.f, seen1 = 0.f;
#pragma unroll
                for (int r = 0; r < RPL; r += 4) {
                    const float4 u = *reinterpret_cast<const float4*>(uv + r);
                    seen0 = fmaf(u.x, s_reg[r], seen0);
                    seen1 = fmaf(u.y, s_reg[r + 1], seen1);
                    seen0 = fmaf(u.z, s_reg[r + 2], seen0);
                    seen1 = fmaf(u.w, s_reg[r + 3], seen1);
                }
                float seen = seen0 + seen1;
#pragma unroll
                for (int m = 1; m < LANES; m <<= 1) seen += __shfl_xor_sync(0xffffffffu, seen, m);
#pragma unroll
                for (int r = 0; r < RPL; r += 4) {
                    const float4 w = *reinterpret_cast<const float4*>(wv + r), au = *reinterpret_cast<const float4*>(auv + r);
                    const float2 ka = __bfloat1622float2(k2[r / 2]), kb = __bfloat1622float2(k2[r / 2 + 1]);
                    const float2 qa = __bfloat1622float2(r2[r / 2]), qb = __bfloat1622float2(r2[r / 2 + 1]);
                    s_reg[r] = fmaf(w.x, s_reg[r], fmaf(ka.x, v, -au.x * seen));          o0 = fmaf(s_reg[r], qa.x, o0);
                    s_reg[r + 1] = fmaf(w.y, s_reg[r + 1], fmaf(ka.y, v, -au.y * seen));  o1 = fmaf(s_reg[r + 1], qa.y, o1);
                    s_reg[r + 2] = fmaf(w.z, s_reg[r + 2], fmaf(kb.x, v, -au.z * seen));  o0 = fmaf(s_reg[r + 2], qb.x, o0);
                    s_reg[r + 3] = fmaf(w.w, s_reg[r + 3], fmaf(kb.y, v, -au.w * seen));  o1 = fmaf(s_reg[r + 3], qb.y, o1);
                }
            } else {
#pragma unroll
                for (int r = 0; r < RPL; r += 4) {
                    const float4 w = *reinterpret_cast<const float4*>(wv + r);
                    const float2 ka = __bfloat1622float2(k2[r / 2]), kb = __bfloat1622float2(k2[r / 2 + 1]);
                    const float2 qa = __bfloat1622float2(r2[r / 2]), qb = __bfloat1622float2(r2[r / 2 + 1]);
                    const float kv0 = ka.x * v, kv1 = ka.y * v, kv2 = kb.x * v, kv3 = kb.y * v;
                    o0 = fmaf(fmaf(b_reg[r], kv0, s_reg[r]), qa.x, o0);          s_reg[r] = fmaf(w.x, s_reg[r], kv0);
                    o1 = fmaf(fmaf(b_reg[r + 1], kv1, s_reg[r + 1]), qa.y, o1);  s_reg[r + 1] = fmaf(w.y, s_reg[r + 1], kv1);
                    o0 = fmaf(fmaf(b_reg[r + 2], kv2, s_reg[r + 2]), qb.x, o0);  s_reg[r + 2] = fmaf(w.z, s_reg[r + 2], kv2);
                    o1 = fmaf(fmaf(b_reg[r + 3], kv3, s_reg[r + 3]), qb.y, o1);  s_reg[r + 3] = fmaf(w.w, s_reg[r + 3], kv3);
                }
            }
            o_part[tt] = o0 + o1;
        }
#pragma unroll
        for (int m = 1; m < LANES; m <<= 1)
#pragma unroll
            for (int tt = 0; tt < TOK; ++tt) o_part[tt] += __shfl_xor_sync(0xffffffffu, o_part[tt], m);
        if (sub == 0 && col)
#pragma unroll
            for (int tt = 0; tt < TOK; ++tt)
                if (tt < n_tok) out[(size_t)(t + tt) * ldo + h * vdim + j0 + cj] = o_part[tt];
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = sub * RPL + r;
        if (col && i < dim) S[(size_t)(j0 + cj) * dim + i] = s_reg[r];
    }
}

// proj [T, ld]: r, k (n_heads x dim) and v (n_heads x vdim) from the given columns; decay [T, ldd] float32
// (n_heads x dim), for float32 rows their logarithms (what the prepare kernel leaves in either case); kind 0 (delta rule): unit [T, ldu] float32 = [u | a * u]; kind 1: bonus [n_heads x dim]
// float32 or null; state [slots, n_heads, vdim, dim] float32 (a value column's key rows lie together, so that the eight
// lanes of a column read and write it in one piece); out [T, ldo] float32 (n_heads x vdim).
SSB_API int ssb_matrix_state_scan(const void* proj, int ld, int dtype, int r_off, int k_off, int v_off,
                                  const float* decay, int ldd, int kind, const float* unit, int ldu, const float* bonus,
                                  float* state, const int* cu_new, const int* seq_slot, float* out, int ldo, int n_seqs,
                                  int n_heads, int dim, int vdim, int pdl, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (dim <= 0 || dim > 256 || vdim <= 0 || n_heads <= 0 || (kind != 0 && kind != 1)) return SSB_ERR_BAD_SIZE;
    if (kind == 0 && unit == nullptr) return SSB_ERR_BAD_SIZE;
    const dim3 grid(n_seqs, n_heads, (vdim + MS_COLS - 1) / MS_COLS);
    if (grid.y > 65535 || grid.z > 65535) return SSB_ERR_BAD_SIZE;
    int rc = 0;
    // bfloat16 rows whose pieces of 16 bytes are aligned take the cp.async form
    const bool pieces = dtype == SSB_BF16 && dim % 8 == 0 && dim <= 128 && vdim % 8 == 0 && ld % 8 == 0 && r_off % 8 == 0 &&
                        k_off % 8 == 0 && v_off % 8 == 0 && ldd % 4 == 0 && (kind != 0 || ldu % 4 == 0) &&
                        !(((uintptr_t)proj | (uintptr_t)decay | (uintptr_t)unit) & 15);
    if (pieces) {
#define SSB_MSA(LANES, RPL, DELTA) do { \
        constexpr int cols = MS_THREADS / LANES; \
        constexpr int stage = ((DELTA ? 3 : 1) * MS_TOKENS * LANES * RPL * 4) + 2 * MS_TOKENS * LANES * RPL * 2 + MS_TOKENS * cols * 2; \
        auto kern = matrix_state_scan_async_kernel<LANES, RPL, DELTA>; \
        if (4 * stage > 48 * 1024) { \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * stage); \
            if (e != cudaSuccess) return (int)e; \
        } \
        const dim3 g2(n_seqs, n_heads, (vdim + cols - 1) / cols); \
        rc = ssb_launch(kern, g2, dim3(MS_THREADS), (size_t)4 * stage, stream, pdl != 0, (const bf16*)proj, ld, r_off, k_off, v_off, \
                        decay, ldd, unit, ldu, bonus, state, cu_new, seq_slot, out, ldo, n_heads, dim, vdim); \
    } while (0)
#define SSB_MSA_DIM(DELTA) do { \
        if (dim <= 32) SSB_MSA(8, 4, DELTA); \
        else if (dim <= 64) SSB_MSA(16, 4, DELTA); \
        else SSB_MSA(16, 8, DELTA); \
    } while (0)
        if (kind == 0) SSB_MSA_DIM(true); else SSB_MSA_DIM(false);
#undef SSB_MSA_DIM
#undef SSB_MSA
        return rc ? rc : ssb_launch_status();
    }
#define SSB_MS(T, RPL, DELTA) \
    rc = ssb_launch(matrix_state_scan_kernel<T, RPL, DELTA>, grid, dim3(MS_THREADS), 0, stream, pdl != 0, (const T*)proj, ld, \
                    r_off, k_off, v_off, decay, ldd, unit, ldu, bonus, state, cu_new, seq_slot, out, ldo, n_heads, dim, vdim)
#define SSB_MS_DIM(T, DELTA) do { \
        if (dim <= 32) SSB_MS(T, 4, DELTA); \
        else if (dim <= 64) SSB_MS(T, 8, DELTA); \
        else if (dim <= 128) SSB_MS(T, 16, DELTA); \
        else SSB_MS(T, 32, DELTA); \
    } while (0)
    if (dtype == SSB_F32) { if (kind == 0) SSB_MS_DIM(float, true); else SSB_MS_DIM(float, false); }
    else if (dtype == SSB_BF16) { if (kind == 0) SSB_MS_DIM(bf16, true); else SSB_MS_DIM(bf16, false); }
    else return SSB_ERR_BAD_DTYPE;
#undef SSB_MS_DIM
#undef SSB_MS
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// One token a sequence (a decode step), bfloat16 projections: what `state_scan_prepare`, the walk and
// `head_norm_gate` do in three launches, in one.  A block takes a sequence and a head: it makes the head's decays
// (and unit key and removal vector) in shared memory, walks the state's value columns 16 at a time (eight lanes a
// column as in the walk above, the state read and written once), and norms and gates the head's output.
// ---------------------------------------------------------------------------------------
template <int RPL, bool DELTA>
__global__ void __launch_bounds__(MS_THREADS)
matrix_state_step_kernel(const bf16* __restrict__ proj, int ld, int r_off, int k_off, int v_off, int g_off, int a_off,
                         const float* __restrict__ z, int ldz, const float* __restrict__ z_bias, int decay_kind,
                         float decay_scale, const float* __restrict__ a_bias, float unit_eps,
                         const float* __restrict__ bonus, float* __restrict__ state, const int* __restrict__ cu_new,
                         const int* __restrict__ seq_slot, const bf16* __restrict__ norm_w, int w_stride, float eps,
                         int gate_kind, bf16* __restrict__ y, int ldy, int n_heads, int dim, int vdim) {
    constexpr int DIMP = MS_LANES * RPL;
    extern __shared__ __align__(16) float st_smem[];
    float* w_s = st_smem;                                // [DIMP] each: decay, key, receptance, unit key, removal
    float* k_s = w_s + DIMP;
    float* r_s = k_s + DIMP;
    float* u_s = r_s + DIMP;
    float* au_s = u_s + DIMP;
    float* o_s = au_s + DIMP;                            // [vdim] the head's output
    __shared__ float red[MS_THREADS / 32];
    const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, sub = tid % MS_LANES, cj = tid / MS_LANES;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const size_t t = (size_t)cu_new[b];
    const bf16* row = proj + t * ld;
    float ksq = 0.f;
    for (int i = tid; i < DIMP; i += MS_THREADS) {
        float w = 0.f, k = 0.f, r = 0.f;
        if (i < dim) {
            const float zv = z[t * ldz + h * dim + i] + z_bias[h * dim + i];
            w = expf(decay_kind == 0 ? -expf(zv) : -decay_scale / (1.0f + expf(-zv)));
            k = __bfloat162float(row[k_off + h * dim + i]);
            r = __bfloat162float(row[r_off + h * dim + i]);
        }
        w_s[i] = w;
        k_s[i] = k;
        r_s[i] = r;
        ksq = fmaf(k, k, ksq);
    }
    if (DELTA) {
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) ksq += __shfl_xor_sync(0xffffffffu, ksq, m);
        if ((tid & 31) == 0) red[tid >> 5] = ksq;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int wv = 0; wv < MS_THREADS / 32; ++wv) tot += red[wv];
        const float inv = 1.0f / sqrtf(tot + unit_eps);
        for (int i = tid; i < DIMP; i += MS_THREADS) {
            float u = 0.f, au = 0.f;
            if (i < dim) {
                u = k_s[i] * inv;
                au = u / (1.0f + expf(-(__bfloat162float(row[a_off + h * dim + i]) + a_bias[h * dim + i])));
            }
            u_s[i] = u;
            au_s[i] = au;
        }
    }
    __syncthreads();
    float* S = state + ((size_t)slot * n_heads + h) * dim * vdim;
    float b_reg[RPL];
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = sub * RPL + r;
        b_reg[r] = (!DELTA && bonus != nullptr && i < dim) ? bonus[h * dim + i] : 0.f;
    }
    // several tiles of 16 columns at a time, all their state on its way before the first is worked on
    constexpr int GROUP = RPL <= 8 ? 4 : RPL == 16 ? 2 : 1;
    for (int j0 = 0; j0 < vdim; j0 += GROUP * MS_COLS) {
        float s_all[GROUP][RPL], v_all[GROUP];
#pragma unroll
        for (int gi = 0; gi < GROUP; ++gi) {
            const int c = j0 + gi * MS_COLS + cj;
            const bool col = c < vdim;
#pragma unroll
            for (int r = 0; r < RPL; ++r) {
                const int i = sub * RPL + r;
                s_all[gi][r] = (col && i < dim) ? S[(size_t)c * dim + i] : 0.f;
            }
            v_all[gi] = col ? __bfloat162float(row[v_off + h * vdim + c]) : 0.f;
        }
#pragma unroll
        for (int gi = 0; gi < GROUP; ++gi) {
            const int c = j0 + gi * MS_COLS + cj;
            const bool col = c < vdim;
            float* s_reg = s_all[gi];
            const float v = v_all[gi];
            float o = 0.f;
            if (DELTA) {
                float seen = 0.f;
#pragma unroll
                for (int r = 0; r < RPL; ++r) seen = fmaf(u_s[sub * RPL + r], s_reg[r], seen);
                seen += __shfl_xor_sync(0xffffffffu, seen, 1);
                seen += __shfl_xor_sync(0xffffffffu, seen, 2);
                seen += __shfl_xor_sync(0xffffffffu, seen, 4);
#pragma unroll
                for (int r = 0; r < RPL; ++r) {
                    const int i = sub * RPL + r;
                    s_reg[r] = fmaf(w_s[i], s_reg[r], fmaf(k_s[i], v, -au_s[i] * seen));
                    o = fmaf(s_reg[r], r_s[i], o);
                }
            } else {
#pragma unroll
                for (int r = 0; r < RPL; ++r) {
                    const int i = sub * RPL + r;
                    const float kv = k_s[i] * v;
                    o = fmaf(fmaf(b_reg[r], kv, s_reg[r]), r_s[i], o);
                    s_reg[r] = fmaf(w_s[i], s_reg[r], kv);
                }
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);
            if (col) {
                if (sub == 0) o_s[c] = o;
#pragma unroll
                for (int r = 0; r < RPL; ++r) {
                    const int i = sub * RPL + r;
                    if (i < dim) S[(size_t)c * dim + i] = s_reg[r];
                }
            }
        }
    }
    __syncthreads();
    // the head's output over its root mean square, weighted and gated
    float part = 0.f;
    for (int c = tid; c < vdim; c += MS_THREADS) part = fmaf(o_s[c], o_s[c], part);
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
    __syncthreads();                                     // red is read above by everyone before it is written again
    if ((tid & 31) == 0) red[tid >> 5] = part;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int wv = 0; wv < MS_THREADS / 32; ++wv) tot += red[wv];
    const float inv = 1.0f / sqrtf(tot / (float)vdim + eps);
    for (int c = tid; c < vdim; c += MS_THREADS) {
        const float gv = __bfloat162float(row[g_off + h * vdim + c]);
        const float sg = 1.0f / (1.0f + expf(-gv));
        const float ga = gate_kind == 0 ? gv * sg : gate_kind == 1 ? sg : gv;
        y[t * ldy + h * vdim + c] = __float2bfloat16_rn(o_s[c] * inv * __bfloat162float(norm_w[(size_t)h * w_stride + c]) * ga);
    }
}

SSB_API int ssb_matrix_state_step(const void* proj, int ld, int r_off, int k_off, int v_off, int g_off, int a_off,
                                  const float* z, int ldz, const float* z_bias, int decay_kind, float decay_scale,
                                  const float* a_bias, float unit_eps, int kind, const float* bonus, float* state,
                                  const int* cu_new, const int* seq_slot, const void* norm_w, int w_stride, float eps,
                                  int gate_kind, void* y, int ldy, int n_seqs, int n_heads, int dim, int vdim, int pdl,
                                  cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (dim <= 0 || dim > 256 || vdim <= 0 || n_heads <= 0 || n_heads > 65535 || (kind != 0 && kind != 1) ||
        decay_kind < 0 || decay_kind > 1 || gate_kind < 0 || gate_kind > 2 || (kind == 0 && a_bias == nullptr))
        return SSB_ERR_BAD_SIZE;
    const dim3 grid(n_seqs, n_heads);
    int rc = 0;
#define SSB_ST(RPL, DELTA) \
    rc = ssb_launch(matrix_state_step_kernel<RPL, DELTA>, grid, dim3(MS_THREADS), (size_t)(5 * MS_LANES * RPL + vdim) * sizeof(float), \
                    stream, pdl != 0, (const bf16*)proj, ld, r_off, k_off, v_off, g_off, a_off, z, ldz, z_bias, decay_kind, \
                    decay_scale, a_bias, unit_eps, bonus, state, cu_new, seq_slot, (const bf16*)norm_w, w_stride, eps, gate_kind, \
                    (bf16*)y, ldy, n_heads, dim, vdim)
#define SSB_ST_DIM(DELTA) do { \
        if (dim <= 32) SSB_ST(4, DELTA); \
        else if (dim <= 64) SSB_ST(8, DELTA); \
        else if (dim <= 128) SSB_ST(16, DELTA); \
        else SSB_ST(32, DELTA); \
    } while (0)
    if (vdim > 8192) return SSB_ERR_BAD_SIZE;
    if (kind == 0) SSB_ST_DIM(true); else SSB_ST_DIM(false);
#undef SSB_ST_DIM
#undef SSB_ST
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// The real-gated linear recurrent unit: a state value per channel,
//     r = sigmoid(g_r + b_r), i = sigmoid(g_i + b_i), log a = rate * r (rate = -8 softplus(lambda) < 0),
//     S_t = a S_(t-1) + sqrt(1 - a^2) * i * u_t,        out_t = S_t * gelu_tanh(y_t + y_bias)
// gates [T, ldg] float32 holds, per block of `block` channels, [g_r (block) | g_i (block)].
// One thread per (sequence, channel), four tokens fetched ahead.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(128)
gated_unit_scan_kernel(const float* __restrict__ gates, int ldg, const float* __restrict__ bias_r,
                       const float* __restrict__ bias_i, const float* __restrict__ rate, const T* __restrict__ u,
                       int ldu, const T* __restrict__ y, int ldy, const float* __restrict__ y_bias,
                       float* __restrict__ state, const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                       T* __restrict__ out, int ldo, int channels, int block) {
    constexpr int AHEAD = 4;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int b = blockIdx.x, c = blockIdx.y * 128 + threadIdx.x;
    const int slot = seq_slot[b];
    if (slot < 0 || c >= channels) return;
    const int t0 = cu_new[b], t1 = cu_new[b + 1];
    const int gc = (c / block) * 2 * block + c % block;           // where the channel's g_r sits; g_i is `block` on
    const float br = bias_r[c], bi = bias_i[c], rt = rate[c], yb = y_bias ? y_bias[c] : 0.f;
    // the float32 path carries the state of a step's tokens in double (it is stored as float32 between steps),
    // and takes the decay and the input's share in double too: a state that remembers for a thousand tokens
    // has a decay within 1e-3 of one, whose float32 rounding is a 1e-4 of its logarithm
    using A = typename std::conditional<std::is_same<T, float>::value, double, float>::type;
    A S = state[(size_t)slot * channels + c];
    float gr[AHEAD], gi[AHEAD], uu[AHEAD], yy[AHEAD];
    auto fetch = [&](int t) {
#pragma unroll
        for (int n = 0; n < AHEAD; ++n)
            if (t + n < t1) {
                const size_t row = (size_t)(t + n);
                gr[n] = gates[row * ldg + gc];
                gi[n] = gates[row * ldg + gc + block];
                uu[n] = ssb_to_float(u[row * ldu + c]);
                yy[n] = ssb_to_float(y[row * ldy + c]);
            }
    };
    fetch(t0);
    for (int t = t0; t < t1; t += AHEAD) {
        float cgr[AHEAD], cgi[AHEAD], cu[AHEAD], cy[AHEAD];
#pragma unroll
        for (int n = 0; n < AHEAD; ++n) { cgr[n] = gr[n]; cgi[n] = gi[n]; cu[n] = uu[n]; cy[n] = yy[n]; }
        if (t + AHEAD < t1) fetch(t + AHEAD);
#pragma unroll
        for (int n = 0; n < AHEAD; ++n)
            if (t + n < t1) {
                if (std::is_same<T, float>::value) {
                    const double r = 1.0 / (1.0 + exp(-((double)cgr[n] + br)));
                    const double i = 1.0 / (1.0 + exp(-((double)cgi[n] + bi)));
                    const double log_a = (double)rt * r;
                    S = fma(exp(log_a), (double)S, sqrt(-expm1(2.0 * log_a)) * i * cu[n]);
                } else {
                    const float r = 1.0f / (1.0f + expf(-(cgr[n] + br)));
                    const float i = 1.0f / (1.0f + expf(-(cgi[n] + bi)));
                    const float log_a = rt * r;
                    S = fmaf(expf(log_a), (float)S, sqrtf(-expm1f(2.0f * log_a)) * i * cu[n]);
                }
                out[(size_t)(t + n) * ldo + c] = ssb_from_float<T>((float)S * gelu_tanh_f(cy[n] + yb));
            }
    }
    state[(size_t)slot * channels + c] = (float)S;
}

// The same recurrence in several launches, for long runs of new tokens in the 16-bit path: everything that does not
// depend on the state (the two gates, a, the input's share, the activation of y) is taken for all tokens at once,
// a and the share written over g_r and g_i and gelu_tanh(y + y_bias) over y; the walk over the tokens is then one
// multiply-add and one product a token.
__global__ void __launch_bounds__(256)
gated_unit_prepare_kernel(float* __restrict__ gates, int ldg, const float* __restrict__ bias_r,
                          const float* __restrict__ bias_i, const float* __restrict__ rate, const bf16* __restrict__ u,
                          int ldu, bf16* __restrict__ y, int ldy, const float* __restrict__ y_bias, int channels, int block,
                          size_t total) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= total) return;
    const size_t row = idx / channels;
    const int c = (int)(idx % channels);
    const int gc = (c / block) * 2 * block + c % block;
    float* g = gates + row * ldg + gc;
    const float r = 1.0f / (1.0f + expf(-(g[0] + bias_r[c])));
    const float i = 1.0f / (1.0f + expf(-(g[block] + bias_i[c])));
    const float log_a = rate[c] * r;
    g[0] = expf(log_a);
    g[block] = sqrtf(-expm1f(2.0f * log_a)) * i * __bfloat162float(u[row * ldu + c]);
    bf16* yp = y + row * ldy + c;
    *yp = __float2bfloat16_rn(gelu_tanh_f(__bfloat162float(*yp) + (y_bias ? y_bias[c] : 0.f)));
}

// The walk itself, over chunks of a sequence's tokens in parallel (S_t = a_t S_(t-1) + s_t composes: a chunk is
// S_out = A S_in + B with A the product of its a and B its own walk from zero).
//   PHASE 0: every (sequence, chunk, channel) walks its chunk from zero and leaves (A, B) in scratch;
//   PHASE 1: every (sequence, channel) walks the chunks in order from the slot's state, leaves each chunk's S_in in
//            scratch and the last S_out in the state;
//   PHASE 2: every (sequence, chunk, channel) walks its chunk from S_in and writes the outputs S_t * y_t.
template <int PHASE>
__global__ void __launch_bounds__(64)
gated_unit_walk_kernel(const float* __restrict__ gates, int ldg, const bf16* __restrict__ y, int ldy,
                       float* __restrict__ state, const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                       bf16* __restrict__ out, int ldo, int channels, int block, int chunk, int max_chunks,
                       float2* __restrict__ scratch) {
    constexpr int AHEAD = 8;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int b = blockIdx.x, c = blockIdx.y * 64 + threadIdx.x, ck = blockIdx.z;
    const int slot = seq_slot[b];
    if (slot < 0 || c >= channels) return;
    const int s0 = cu_new[b], s1 = cu_new[b + 1];
    float2* mine = scratch + ((size_t)b * max_chunks) * channels + c;      // [chunk][channel]
    if (PHASE == 1) {
        const int n = (s1 - s0 + chunk - 1) / chunk;
        float S = state[(size_t)slot * channels + c];
        for (int k = 0; k < n; ++k) {
            const float2 ab = mine[(size_t)k * channels];
            mine[(size_t)k * channels].x = S;
            S = fmaf(ab.x, S, ab.y);
        }
        state[(size_t)slot * channels + c] = S;
        return;
    }
    const int t0 = s0 + ck * chunk, t1 = min(s1, t0 + chunk);
    if (t0 >= t1) return;
    const int gc = (c / block) * 2 * block + c % block;
    float S = PHASE == 2 ? mine[(size_t)ck * channels].x : 0.f, A = 1.f;
    float a[AHEAD], sh[AHEAD], yy[AHEAD];
    auto fetch = [&](int t) {
#pragma unroll
        for (int n = 0; n < AHEAD; ++n)
            if (t + n < t1) {
                const size_t row = (size_t)(t + n);
                a[n] = gates[row * ldg + gc];
                sh[n] = gates[row * ldg + gc + block];
                if (PHASE == 2) yy[n] = __bfloat162float(y[row * ldy + c]);
            }
    };
    fetch(t0);
    for (int t = t0; t < t1; t += AHEAD) {
        float ca[AHEAD], cs[AHEAD], cy[AHEAD];
#pragma unroll
        for (int n = 0; n < AHEAD; ++n) { ca[n] = a[n]; cs[n] = sh[n]; cy[n] = PHASE == 2 ? yy[n] : 0.f; }
        if (t + AHEAD < t1) fetch(t + AHEAD);
#pragma unroll
        for (int n = 0; n < AHEAD; ++n)
            if (t + n < t1) {
                S = fmaf(ca[n], S, cs[n]);
                if (PHASE == 0) A *= ca[n];
                else out[(size_t)(t + n) * ldo + c] = __float2bfloat16_rn(S * cy[n]);
            }
    }
    if (PHASE == 0) mine[(size_t)ck * channels] = make_float2(A, S);
}

constexpr int GU_CHUNK = 128;
SSB_API long long ssb_gated_unit_scan_scratch(int n_seqs, int max_new, int channels) {
    return 2ll * n_seqs * ((max_new + GU_CHUNK - 1) / GU_CHUNK) * channels;          // floats
}

SSB_API int ssb_gated_unit_scan_split(float* gates, int ldg, const float* bias_r, const float* bias_i, const float* rate,
                                      const void* u, int ldu, void* y, int ldy, const float* y_bias, float* state,
                                      const int* cu_new, const int* seq_slot, void* out, int ldo, int n_seqs, int n_tokens,
                                      int max_new, int channels, int block, float* scratch, int pdl, cudaStream_t stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (channels <= 0 || block <= 0 || channels % block || max_new <= 0 || !scratch || ((uintptr_t)scratch & 7)) return SSB_ERR_BAD_SIZE;
    const size_t total = (size_t)n_tokens * channels;
    int rc = ssb_launch(gated_unit_prepare_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, pdl != 0, gates,
                        ldg, bias_r, bias_i, rate, (const bf16*)u, ldu, (bf16*)y, ldy, y_bias, channels, block, total);
    if (!rc) rc = ssb_launch_status();
    if (rc) return rc;
    const int chunks = (max_new + GU_CHUNK - 1) / GU_CHUNK;
    const dim3 grid(n_seqs, (channels + 63) / 64, chunks);
    if (grid.y > 65535 || grid.z > 65535) return SSB_ERR_BAD_SIZE;
#define SSB_GU(PHASE, GRID) \
    rc = ssb_launch(gated_unit_walk_kernel<PHASE>, GRID, dim3(64), 0, stream, pdl != 0, (const float*)gates, ldg, (const bf16*)y, \
                    ldy, state, cu_new, seq_slot, (bf16*)out, ldo, channels, block, GU_CHUNK, chunks, (float2*)scratch); \
    if (!rc) rc = ssb_launch_status(); \
    if (rc) return rc
    SSB_GU(0, grid);
    SSB_GU(1, dim3(n_seqs, (channels + 63) / 64));
    SSB_GU(2, grid);
#undef SSB_GU
    return 0;
}

SSB_API int ssb_gated_unit_scan(const float* gates, int ldg, const float* bias_r, const float* bias_i, const float* rate,
                                const void* u, int ldu, const void* y, int ldy, const float* y_bias, float* state,
                                const int* cu_new, const int* seq_slot, void* out, int ldo, int dtype, int n_seqs,
                                int channels, int block, int pdl, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (channels <= 0 || block <= 0 || channels % block) return SSB_ERR_BAD_SIZE;
    const dim3 grid(n_seqs, (channels + 127) / 128);
    if (grid.y > 65535) return SSB_ERR_BAD_SIZE;
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(gated_unit_scan_kernel<float>, grid, dim3(128), 0, stream, pdl != 0, gates, ldg, bias_r, bias_i, rate,
                        (const float*)u, ldu, (const float*)y, ldy, y_bias, state, cu_new, seq_slot, (float*)out, ldo,
                        channels, block);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(gated_unit_scan_kernel<bf16>, grid, dim3(128), 0, stream, pdl != 0, gates, ldg, bias_r, bias_i, rate,
                        (const bf16*)u, ldu, (const bf16*)y, ldy, y_bias, state, cu_new, seq_slot, (bf16*)out, ldo,
                        channels, block);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}
