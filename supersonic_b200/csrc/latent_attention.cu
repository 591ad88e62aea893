// Latent attention on the tensor cores (mma.sync m16n8k16), prompts and decode steps alike.
//
// Every head of a token attends over the same cached rows [latent (dv) | rotated key part]
// (dk elements; the values are the first dv of them), so a block takes 32 (token, head) rows of
// one sequence and streams that sequence's pages once for all of them: a page (64 keys) arrives
// in shared memory through a two-stage cp.async ring and serves as K for the scores and, read
// transposed, as V for the weighted sum.  The warps of a block are RG groups of 16 rows times KW
// slices: of the page's keys for the scores (16 or 8 keys each), of the value width for the sum.
// Prompts run two row groups (32 rows a block); a decode step of up to 16 heads runs one row group
// with eight slices, so that all eight warps share the one tile of rows that exists.  Scores, maxima, weights and sums are float32; a weight enters the second product as
// the sum of two bfloat16 numbers (p = hi + lo, two MMAs), so that it keeps 16 bits of mantissa.
// The softmax may carry a sink per head (one more term in the denominator).  A decode step can cut a
// sequence's pages into splits (blockIdx.z) whose partial results a second kernel merges.
#include "mma_helpers.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

constexpr int LA_BN = 64;            // keys a turn: one page
constexpr int LA_PLD = LA_BN + 8;    // padded row of the weights' tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr int LA_PROMPT_FORM = 2;    // the form prompts take (2: two row groups x four slices; 3: x eight slices)

template <int MAXU, int RG, int KW>
__global__ void __launch_bounds__(RG * KW * 32)
latent_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache, const int* __restrict__ cu_new,
                        const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                        const int* __restrict__ page_table, int max_pages, bf16* __restrict__ out,
                        float* __restrict__ partial, const float* __restrict__ sinks, int n_heads, int dk, int dv,
                        int window, float scale_log2, int n_splits) {
    constexpr int LA_ROWS = 16 * RG, LA_THREADS = RG * KW * 32;      // (token, head) rows a block
    constexpr int KS = LA_BN / KW, NJ = KS / 8;                      // keys a slice, 8-key tiles a slice
    extern __shared__ __align__(16) unsigned char smem[];
    const int ldk = dk + 8;
    bf16* q_s = reinterpret_cast<bf16*>(smem);
    bf16* k_s = q_s + LA_ROWS * ldk;
    bf16* p_hi = k_s + 2 * LA_BN * ldk;
    bf16* p_lo = p_hi + LA_ROWS * LA_PLD;
    float* m_part = reinterpret_cast<float*>(p_lo + LA_ROWS * LA_PLD);
    float* l_part = m_part + LA_ROWS * KW;

    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int b = blockIdx.y, slot = seq_slot[b];
    if (slot < 0) return;                                             // padding row
    const int t0 = cu_new[b], n_rows = (cu_new[b + 1] - t0) * n_heads, start = seq_start[b];
    const int row0 = blockIdx.x * LA_ROWS;
    if (row0 >= n_rows) return;
    const int rows_here = min(LA_ROWS, n_rows - row0);
    const int pos_first = start + row0 / n_heads, pos_last = start + (row0 + rows_here - 1) / n_heads;
    const int kb_lo = window > 0 ? max(0, pos_first - window + 1) >> 6 : 0, kb_hi = pos_last >> 6;
    const int per = (kb_hi - kb_lo + n_splits) / n_splits;
    const int my_lo = kb_lo + (int)blockIdx.z * per, my_hi = min(kb_hi, my_lo + per - 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rg = warp / KW, kw = warp % KW, g = lane >> 2, t = lane & 3;
    const size_t grow0 = (size_t)t0 * n_heads + row0;                 // first row among all (token, head) rows
    const int units = dv >> 4, U = (units + KW - 1) / KW, u0 = kw * U;
    const int n_mine = max(0, min(U, units - u0));

    if (my_lo > my_hi) {                                              // a split without pages: says so and leaves
        if (tid < rows_here) {
            float* pr = partial + ((grow0 + tid) * n_splits + blockIdx.z) * (size_t)(dv + 2);
            pr[0] = -INFINITY;
            pr[1] = 0.f;
        }
        return;
    }
    const int* pt = page_table + (size_t)slot * max_pages;
    const int chunks = dk >> 3;
    {   // the block's query rows, zero beyond the sequence's rows
        const bf16* src = q + grow0 * dk;
        for (int c = tid; c < LA_ROWS * chunks; c += LA_THREADS) {
            const int r = c / chunks, ch = c % chunks;
            bf16* dst = q_s + r * ldk + ch * 8;
            if (r < rows_here) cp_async16((uint32_t)__cvta_generic_to_shared(dst), src + (size_t)r * dk + ch * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
    auto load_page = [&](int kb, int stage) {
        const bf16* src = cache + (size_t)pt[kb] * LA_BN * dk;
        bf16* dst = k_s + stage * LA_BN * ldk;
        for (int c = tid; c < LA_BN * chunks; c += LA_THREADS) {
            const int r = c / chunks, ch = c % chunks;
            cp_async16((uint32_t)__cvta_generic_to_shared(dst + r * ldk + ch * 8), src + (size_t)r * dk + ch * 8);
        }
        cp_async_commit();
    };
    load_page(my_lo, 0);

    int pos_r[2];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = rg * 16 + g + i * 8;
        pos_r[i] = r < rows_here ? start + (row0 + r) / n_heads : -1;
    }
    float acc[MAXU][2][4];
#pragma unroll
    for (int u = 0; u < MAXU; ++u)
#pragma unroll
        for (int j = 0; j < 2; ++j) acc[u][j][0] = acc[u][j][1] = acc[u][j][2] = acc[u][j][3] = 0.f;
    const uint32_t qb = (uint32_t)__cvta_generic_to_shared(q_s);
    const uint32_t phb = (uint32_t)__cvta_generic_to_shared(p_hi), plb = (uint32_t)__cvta_generic_to_shared(p_lo);

    for (int kb = my_lo; kb <= my_hi; ++kb) {
        const int stage = (kb - my_lo) & 1;
        cp_async_wait<0>();
        __syncthreads();                                              // page kb has landed; everyone is done with kb - 1
        if (kb < my_hi) load_page(kb + 1, stage ^ 1);                 // ... so its stage and the weights' tile are free
        const uint32_t kbase = (uint32_t)__cvta_generic_to_shared(k_s + stage * LA_BN * ldk);

        // scores of this warp's 16 rows on its KS keys
        float s[NJ][4];
#pragma unroll
        for (int j = 0; j < NJ; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        {
            const uint32_t qa = qb + ((rg * 16 + (lane & 15)) * ldk + (lane >> 4) * 8) * 2;
            // B fragments: 16 keys (two tiles, ldmatrix.x4) or 8 keys (one tile, ldmatrix.x2: lanes 0-15 give addresses)
            const uint32_t ka = NJ == 2
                ? kbase + ((kw * 16 + ((lane >> 4) << 3) + (lane & 7)) * ldk + ((lane >> 3) & 1) * 8) * 2
                : kbase + ((kw * 8 + (lane & 7)) * ldk + ((lane >> 3) & 1) * 8) * 2;
#pragma unroll 4
            for (int ks = 0; ks < (dk >> 4); ++ks) {
                uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                ldmatrix_x4(qa + ks * 32, a0, a1, a2, a3);
                if (NJ == 2) {
                    ldmatrix_x4(ka + ks * 32, b0, b1, b2, b3);
                    mma16816(s[0], a0, a1, a2, a3, b0, b1);
                    mma16816(s[NJ - 1], a0, a1, a2, a3, b2, b3);
                } else {
                    ldmatrix_x2(ka + ks * 32, b0, b1);
                    mma16816(s[0], a0, a1, a2, a3, b0, b1);
                }
            }
        }
        const int key0 = kb * LA_BN + kw * KS;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < NJ; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = e >> 1, key = key0 + j * 8 + 2 * t + (e & 1);
                const bool seen = key <= pos_r[i] && (window <= 0 || key > pos_r[i] - window);
                const float v = seen ? s[j][e] * scale_log2 : -INFINITY;
                s[j][e] = v;
                mx[i] = fmaxf(mx[i], v);
            }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            if (t == 0) m_part[(rg * 16 + g + i * 8) * KW + kw] = mx[i];
        }
        __syncthreads();
        float m_new[2], alpha[2], sum[2] = {0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float* mp = m_part + (rg * 16 + g + i * 8) * KW;
            m_new[i] = m_run[i];
#pragma unroll
            for (int w = 0; w < KW; ++w) m_new[i] = fmaxf(m_new[i], mp[w]);
            alpha[i] = (m_new[i] == -INFINITY) ? 1.f : exp2f(m_run[i] - m_new[i]);
        }
#pragma unroll
        for (int j = 0; j < NJ; ++j)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float p0 = (m_new[i] == -INFINITY) ? 0.f : exp2f(s[j][2 * i] - m_new[i]);
                const float p1 = (m_new[i] == -INFINITY) ? 0.f : exp2f(s[j][2 * i + 1] - m_new[i]);
                sum[i] += p0 + p1;
                const __nv_bfloat162 hi = __floats2bfloat162_rn(p0, p1);
                const __nv_bfloat162 lo = __floats2bfloat162_rn(p0 - __low2float(hi), p1 - __high2float(hi));
                const int off = (rg * 16 + g + i * 8) * LA_PLD + kw * KS + j * 8 + 2 * t;
                *reinterpret_cast<__nv_bfloat162*>(p_hi + off) = hi;
                *reinterpret_cast<__nv_bfloat162*>(p_lo + off) = lo;
            }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
            sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
            if (t == 0) l_part[(rg * 16 + g + i * 8) * KW + kw] = sum[i];
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float* lp = l_part + (rg * 16 + g + i * 8) * KW;
            float part = 0.f;
#pragma unroll
            for (int w = 0; w < KW; ++w) part += lp[w];
            l_run[i] = l_run[i] * alpha[i] + part;
            m_run[i] = m_new[i];
        }
        // weighted sum of this warp's slice of the value width
#pragma unroll
        for (int u = 0; u < MAXU; ++u)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                acc[u][j][0] *= alpha[0]; acc[u][j][1] *= alpha[0];
                acc[u][j][2] *= alpha[1]; acc[u][j][3] *= alpha[1];
            }
        const uint32_t pa = ((rg * 16 + (lane & 15)) * LA_PLD + (lane >> 4) * 8) * 2;
        const uint32_t va = kbase + (((((lane >> 3) & 1) << 3) + (lane & 7)) * ldk + (lane >> 4) * 8) * 2;
#pragma unroll
        for (int k2 = 0; k2 < LA_BN / 16; ++k2) {
            uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
            ldmatrix_x4(phb + pa + k2 * 32, h0, h1, h2, h3);
            ldmatrix_x4(plb + pa + k2 * 32, l0, l1, l2, l3);
#pragma unroll
            for (int u = 0; u < MAXU; ++u)
                if (u < n_mine) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(va + (k2 * 16 * ldk + (u0 + u) * 16) * 2, b0, b1, b2, b3);
                    mma16816(acc[u][0], h0, h1, h2, h3, b0, b1);
                    mma16816(acc[u][1], h0, h1, h2, h3, b2, b3);
                    mma16816(acc[u][0], l0, l1, l2, l3, b0, b1);
                    mma16816(acc[u][1], l0, l1, l2, l3, b2, b3);
                }
        }
    }

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = rg * 16 + g + i * 8;
        if (r >= rows_here) continue;
        const size_t grow = grow0 + r;
        if (n_splits > 1) {                                           // unnormalised, for the merge
            float* pr = partial + (grow * n_splits + blockIdx.z) * (size_t)(dv + 2);
            if (kw == 0 && t == 0) { pr[0] = m_run[i]; pr[1] = l_run[i]; }
#pragma unroll
            for (int u = 0; u < MAXU; ++u)
                if (u < n_mine)
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int col = (u0 + u) * 16 + j * 8 + 2 * t;
                        pr[2 + col] = acc[u][j][2 * i];
                        pr[2 + col + 1] = acc[u][j][2 * i + 1];
                    }
            continue;
        }
        float keep = 1.f, l = l_run[i];
        if (sinks != nullptr) {
            const float sk = sinks[(row0 + r) % n_heads] * LOG2E;
            const float m_all = fmaxf(m_run[i], sk);
            keep = (m_run[i] == -INFINITY) ? 0.f : exp2f(m_run[i] - m_all);
            l = l * keep + exp2f(sk - m_all);
        }
        const float inv = l > 0.f ? keep / l : 0.f;
        bf16* dst = out + grow * dv;
#pragma unroll
        for (int u = 0; u < MAXU; ++u)
            if (u < n_mine)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int col = (u0 + u) * 16 + j * 8 + 2 * t;
                    *reinterpret_cast<uint32_t*>(dst + col) = pack2(acc[u][j][2 * i] * inv, acc[u][j][2 * i + 1] * inv);
                }
    }
}

// the splits of a row joined: partial [rows][n_splits][m, l, dv sums], maxima in log2 units
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* __restrict__ partial, const float* __restrict__ sinks,
                              const int* __restrict__ slot_of_row_token, bf16* __restrict__ out, int n_heads,
                              int dv, int n_splits) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const size_t row = blockIdx.x;
    if (slot_of_row_token[row / n_heads] < 0) return;                 // padding row: nothing was written for it
    const float* pr = partial + row * n_splits * (size_t)(dv + 2);
    float m_all = sinks ? sinks[row % n_heads] * LOG2E : -INFINITY;
    for (int z = 0; z < n_splits; ++z) m_all = fmaxf(m_all, pr[(size_t)z * (dv + 2)]);
    float l = sinks ? exp2f(sinks[row % n_heads] * LOG2E - m_all) : 0.f;
    for (int z = 0; z < n_splits; ++z) {
        const float m = pr[(size_t)z * (dv + 2)];
        if (m != -INFINITY) l += pr[(size_t)z * (dv + 2) + 1] * exp2f(m - m_all);
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int c = threadIdx.x; c < dv; c += 128) {
        float a = 0.f;
        for (int z = 0; z < n_splits; ++z) {
            const float m = pr[(size_t)z * (dv + 2)];
            if (m != -INFINITY) a += pr[(size_t)z * (dv + 2) + 2 + c] * exp2f(m - m_all);
        }
        out[row * dv + c] = __float2bfloat16_rn(a * inv);
    }
}

static long long latent_attention_smem(int dk, int rows, int kw) {
    return (long long)(rows + 2 * LA_BN) * (dk + 8) * 2 + 2 * rows * LA_PLD * 2 + 2 * rows * kw * 4;
}

// q [tokens, heads x dk] and out [tokens, heads x dv] contiguous bfloat16; cache [pages][64][dk];
// partial: float32 scratch of tokens x heads x n_splits x (dv + 2) when n_splits > 1
SSB_API int ssb_latent_attention(const void* q, const void* cache, const int* cu_new, const int* seq_start,
                                 const int* seq_slot, const int* slot_of_token, const int* page_table, int max_pages,
                                 void* out, float* partial, const float* sinks, int n_seqs, int max_new, int n_tokens,
                                 int n_heads, int dk, int dv, int page_shift, int window, float scale, int n_splits,
                                 int form, int pdl, cudaStream_t stream) {
    // form: 0 picks by the step (one row group of eight slices when a sequence brings at most 16 rows, else two
    // row groups); 1, 2, 3 ask for (1 x 8), (2 x 4), (2 x 8) row groups x slices
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (page_shift != 6 || dk % 16 || dv % 16 || dv > dk || dv > 512 || dv <= 0 || n_heads <= 0) return SSB_ERR_BAD_SIZE;
    if (((uintptr_t)q | (uintptr_t)cache | (uintptr_t)out) & 15) return SSB_ERR_BAD_SIZE;
    if (n_splits < 1 || n_splits > 65535 || (n_splits > 1 && partial == nullptr)) return SSB_ERR_BAD_SIZE;
    if (form == 0) form = (long long)max_new * n_heads <= 16 ? 1 : LA_PROMPT_FORM;
    if (form < 1 || form > 3) return SSB_ERR_BAD_SIZE;
    const int rows = form == 1 ? 16 : 32, kw = form == 2 ? 4 : 8;
    const long long smem = latent_attention_smem(dk, rows, kw);
    if (smem > 227 * 1024) return SSB_ERR_BAD_SIZE;
    const long long tiles = ((long long)max_new * n_heads + rows - 1) / rows;
    if (tiles > 0x7fffffffll || n_seqs > 65535) return SSB_ERR_BAD_SIZE;
    const dim3 grid((unsigned)tiles, n_seqs, n_splits);
    const int U = (dv / 16 + kw - 1) / kw;
    int rc;
#define SSB_LA(MAXU, RG, KW) do { \
        static long long configured = 0; \
        if (smem > configured) { \
            cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<MAXU, RG, KW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e; \
            configured = smem; \
        } \
        rc = ssb_launch(latent_attention_kernel<MAXU, RG, KW>, grid, dim3(RG * KW * 32), (size_t)smem, stream, pdl != 0, \
                        (const bf16*)q, (const bf16*)cache, cu_new, seq_start, seq_slot, page_table, max_pages, (bf16*)out, \
                        partial, sinks, n_heads, dk, dv, window, scale * LOG2E, n_splits); \
    } while (0)
#define SSB_LA_FORM(RG, KW) do { \
        if (U <= 2) SSB_LA(2, RG, KW); else if (U <= 4) SSB_LA(4, RG, KW); else SSB_LA(8, RG, KW); \
    } while (0)
    if (form == 1) SSB_LA_FORM(1, 8);
    else if (form == 2) SSB_LA_FORM(2, 4);
    else { if (U <= 2) SSB_LA(2, 2, 8); else SSB_LA(4, 2, 8); }
#undef SSB_LA_FORM
#undef SSB_LA
    if (rc) return rc;
    rc = ssb_launch_status();
    if (rc || n_splits == 1) return rc;
    rc = ssb_launch(latent_attention_merge_kernel, dim3((unsigned)((long long)n_tokens * n_heads)), dim3(128), 0, stream,
                    pdl != 0, (const float*)partial, sinks, slot_of_token, (bf16*)out, n_heads, dv, n_splits);
    return rc ? rc : ssb_launch_status();
}
