// From a token's projected row to the heads an attention kernel reads, and
// into the cache: one kernel for mixers whose projections come as one float32
// row per token, [q heads | k heads | (v heads) | (anything else)], at any
// column offsets.
//
//   q and k heads (hd entries each) are either rotated by position (rotate-half
//   layout: entry i < rot/2 is paired with entry i + rot/2; cosine and sine
//   come from tables [positions, rot/2], which may carry a common factor;
//   entries from `rot` on pass; with `paired` the neighbours 2i and 2i + 1 are
//   a pair instead) or, with norm_eps > 0, divided by their root
//   mean square, x / sqrt(mean(x^2) + norm_eps), or left as they are; with
//   `row_inv` (float32 [T, 2]: one factor per token for its whole q row and
//   one for its whole k row, made by row_inv_rms below) and weights over those
//   whole rows, q and k are first multiplied by factor * weight: an RMS norm
//   over the whole projection, before the heads are split and turned;
//   v heads (vd entries each) are copied: from their own columns, or — v_col < 0
//   — from the k columns as projected, before the rotation (vd == hd then).
//
// q goes to q_out [T, nh*hd]; k and v go to the packed outputs (if given) and
// into the paged cache (if given) under the rules of the rotary kernel of
// elementwise.cu: position p of step row b lands in logical page
// p / page_tokens (modulo ring_pages if > 0) at row p % page_tokens; in a ring
// only the last ring_pages*page_tokens positions of a sequence are written;
// a row at or past new_lens of its sequence is padding and is not cached.
//
// Also here: the sigmoid gate on the attention's result and the tanh cap.
#include "common.cuh"

#define HE_MAX_PER_LANE 16    // head widths up to 512

template <typename TC>
__global__ void __launch_bounds__(128)
head_encode_kernel(const float* __restrict__ proj, int ld, int q_col, int k_col, int v_col,
                   const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int rot, float norm_eps,
                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                   const int* __restrict__ new_lens, const int* __restrict__ block_table, int table_width,
                   int ring_pages, int page_tokens, TC* __restrict__ q_out, TC* __restrict__ k_out,
                   TC* __restrict__ v_out, TC* __restrict__ k_pages, TC* __restrict__ v_pages, int nh, int nkv,
                   int hd, int vd, const float* __restrict__ row_inv, const float* __restrict__ q_w,
                   const float* __restrict__ k_w, int paired) {
    // grid (token, groups of four heads), a warp per head: heads 0..nh-1 are q, then nkv k heads, then nkv v heads
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int head = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (head >= nh + 2 * nkv) return;
    const int pos = tok_pos[t];
    const int b = tok_seq[t];
    const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
    const int g = is_q ? head : (is_k ? head - nh : head - nh - nkv);
    const int width = (is_q || is_k) ? hd : vd;
    const float* x = proj + (size_t)t * ld +
                     (is_q ? q_col + g * hd : (is_k ? k_col + g * hd : (v_col >= 0 ? v_col + g * vd : k_col + g * hd)));

    TC* cache = nullptr;
    if (!is_q && k_pages != nullptr) {
        int lp = pos / page_tokens;
        bool keep = pos < new_lens[b];
        if (ring_pages > 0) {
            keep = keep && pos >= new_lens[b] - ring_pages * page_tokens;
            lp %= ring_pages;
        }
        if (keep) {
            const int page = block_table[(size_t)b * table_width + lp];
            const size_t row = ((size_t)page * nkv + g) * page_tokens + (pos % page_tokens);
            cache = is_k ? k_pages + row * hd : v_pages + row * vd;
        }
    }
    TC* dst = is_q ? q_out + ((size_t)t * nh + g) * hd
                   : (is_k ? (k_out ? k_out + ((size_t)t * nkv + g) * hd : nullptr)
                           : (v_out ? v_out + ((size_t)t * nkv + g) * vd : nullptr));
    pdl_wait();
    pdl_launch();
    if (!is_q && !is_k) {                                    // values: a copy
        for (int d = lane; d < width; d += 32) {
            const TC r = from_f32<TC>(x[d]);
            if (dst) dst[d] = r;
            if (cache) cache[d] = r;
        }
        return;
    }
    float inv = 1.f;
    if (norm_eps > 0.f) {
        float ss = 0.f;
        for (int d = lane; d < width; d += 32) ss = fmaf(x[d], x[d], ss);
        ss = warp_sum(ss);
        inv = 1.f / sqrtf(ss / (float)width + norm_eps);
    }
    const float* w = nullptr;                                // the whole-row norm's weights of this head
    if (row_inv) {
        inv = row_inv[2 * t + (is_q ? 0 : 1)];
        w = (is_q ? q_w : k_w) + (size_t)g * hd;
    }
    const int half = rot >> 1;
    if (half > 0) {
        const float* cs = cos_tab + (size_t)pos * half;
        const float* sn = sin_tab + (size_t)pos * half;
        for (int j = lane; j < half; j += 32) {
            const int i0 = paired ? 2 * j : j, i1 = paired ? 2 * j + 1 : j + half;
            float x0 = x[i0] * inv, x1 = x[i1] * inv;
            if (w) { x0 *= w[i0]; x1 *= w[i1]; }
            const float c = cs[j], s = sn[j];
            const TC r0 = from_f32<TC>(x0 * c - x1 * s);
            const TC r1 = from_f32<TC>(x1 * c + x0 * s);
            if (dst) { dst[i0] = r0; dst[i1] = r1; }
            if (cache) { cache[i0] = r0; cache[i1] = r1; }
        }
    }
    for (int d = rot + lane; d < width; d += 32) {
        const TC r = from_f32<TC>(w ? x[d] * inv * w[d] : x[d] * inv);
        if (dst) dst[d] = r;
        if (cache) cache[d] = r;
    }
}

TQ_API int tq_head_encode(const float* proj, int ld, int q_col, int k_col, int v_col, const float* cos_tab,
                          const float* sin_tab, int rot, float norm_eps, const int* tok_pos, const int* tok_seq,
                          const int* new_lens, const int* block_table, int table_width, int ring_pages,
                          int page_tokens, void* q_out, void* k_out, void* v_out, void* k_pages, void* v_pages,
                          int cache_dtype, int n_tokens, int nh, int nkv, int hd, int vd, const float* row_inv,
                          const float* q_w, const float* k_w, int paired, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (row_inv && (!q_w || (nkv > 0 && !k_w) || norm_eps > 0.f)) return (int)cudaErrorInvalidValue;
    if (rot < 0 || rot > hd || (rot & 1) || page_tokens <= 0 || hd <= 0 || vd <= 0) return (int)cudaErrorInvalidValue;
    if (rot > 0 && (!cos_tab || !sin_tab)) return (int)cudaErrorInvalidValue;
    if ((k_pages == nullptr) != (v_pages == nullptr)) return (int)cudaErrorInvalidValue;
    if (k_pages && !block_table) return (int)cudaErrorInvalidValue;
    if (nkv > 0 && v_col < 0 && vd != hd) return (int)cudaErrorInvalidValue;
    const int groups = (nh + 2 * nkv + 3) / 4;
    if (groups > 65535) return (int)cudaErrorInvalidValue;
    const dim3 grid(n_tokens, groups);
#define TQ_LAUNCH(TC)                                                                                              \
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, head_encode_kernel<TC>, grid, dim3(128), 0, stream, proj, ld, q_col,  \
                         k_col, v_col, cos_tab, sin_tab, rot, norm_eps, tok_pos, tok_seq, new_lens, block_table,   \
                         table_width, ring_pages, page_tokens, (TC*)q_out, (TC*)k_out, (TC*)v_out, (TC*)k_pages,   \
                         (TC*)v_pages, nh, nkv, hd, vd, row_inv, q_w, k_w, paired)
    if (cache_dtype == TQ_F32) TQ_LAUNCH(float);
    if (cache_dtype == TQ_BF16) TQ_LAUNCH(bf16);
#undef TQ_LAUNCH
    return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------
// out[t, 0] = 1 / sqrt(sum(q row^2) / q_count + eps), out[t, 1] likewise for the k row (k_n == 0: no k row): the
// factors of an RMS norm over a token's whole q and k projections.  The counts are the rows' true lengths where
// the rows are padded with zeros.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
row_inv_rms_kernel(const float* __restrict__ proj, int ld, int q_col, int q_n, int q_count, int k_col, int k_n,
                   int k_count, float eps, float* __restrict__ out) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    pdl_wait();
    pdl_launch();
    const float* row = proj + (size_t)t * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_n; i += blockDim.x) ss = fmaf(row[q_col + i], row[q_col + i], ss);
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) out[2 * t] = 1.f / sqrtf(ss / (float)q_count + eps);
    if (k_n <= 0) return;
    ss = 0.f;
    for (int i = threadIdx.x; i < k_n; i += blockDim.x) ss = fmaf(row[k_col + i], row[k_col + i], ss);
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) out[2 * t + 1] = 1.f / sqrtf(ss / (float)k_count + eps);
}

TQ_API int tq_row_inv_rms(const float* proj, int ld, int q_col, int q_n, int q_count, int k_col, int k_n, int k_count,
                          float eps, float* out, int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!proj || !out || q_n <= 0 || q_count <= 0 || k_n < 0 || (k_n > 0 && k_count <= 0)) return (int)cudaErrorInvalidValue;
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, row_inv_rms_kernel, dim3(n_tokens), dim3(q_n >= 1024 ? 256 : 128), 0, stream,
                         proj, ld, q_col, q_n, q_count, k_col, k_n, k_count, eps, out);
}

// ---------------------------------------------------------------------------
// x[t, i] *= sigmoid(gate[t * ldg + i]): a gate per entry on the heads side by side.
// ---------------------------------------------------------------------------
template <typename TC>
__global__ void sigmoid_gate_kernel(TC* __restrict__ x, const float* __restrict__ gate, int ldg, int n, size_t total) {
    pdl_wait();
    pdl_launch();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / n;
        const int i = (int)(idx - t * n);
        const float g = gate[t * ldg + i];
        x[idx] = from_f32<TC>(to_f32<TC>(x[idx]) / (1.f + expf(-g)));
    }
}

TQ_API int tq_sigmoid_gate(void* x, int dtype, const float* gate, int ldg, int n_rows, int n, cudaStream_t stream) {
    const size_t total = (size_t)n_rows * n;
    if (total == 0) return 0;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == TQ_F32)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, sigmoid_gate_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0,
                             stream, (float*)x, gate, ldg, n, total);
    if (dtype == TQ_BF16)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, sigmoid_gate_kernel<bf16>, dim3((unsigned)blocks), dim3(threads), 0,
                             stream, (bf16*)x, gate, ldg, n, total);
    return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------
// x <- cap * tanh(x / cap), in place (float32).
// ---------------------------------------------------------------------------
__global__ void tanh_cap_kernel(float* __restrict__ x, size_t total, float cap) {
    pdl_wait();
    pdl_launch();
    const float inv = 1.f / cap;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x)
        x[idx] = cap * tanhf(x[idx] * inv);
}

TQ_API int tq_tanh_cap(float* x, size_t total, float cap, cudaStream_t stream) {
    if (total == 0) return 0;
    if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, tanh_cap_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, total, cap);
}
