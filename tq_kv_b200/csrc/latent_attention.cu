// Attention through a latent: every token is cached as ONE row, the normed latent c (n values) followed by a
// rotated key part k_r (r values) that all heads share.  Head h's key would be [U_k[h] c, k_r] and its value
// U_v[h] c; instead of expanding the cache, the query is carried into the latent's space,
//
//   q~[h] = [U_k[h]^T q_flat[h], rot(q_rot[h])]       (n + r values),    score = q~[h] . [c, k_r] * scale,
//
// the attention kernels run with one shared key/value head whose rows are the cache rows (the value of a row being
// the row itself), and the result, a weighted mean of latents, is expanded afterwards:  o[h] = U_v[h] mean(c).
// The three kernels here are what stands around those attention kernels:
//
//   latent_rows    per token, from the float32 results of the down projections: the RMS-normed query latent (for the
//                  up projection that follows); the cache row [norm(c) * w, rot(k_r), 0 ...] written to the step's
//                  packed rows and / or the sequence's page; rows are padded with zeros to the width `rp` the
//                  attention kernels take
//   latent_query   per (token, head): q~ as above
//   latent_expand  per (token, head): o[h] = U_v[h] mean(c), times sigmoid(gate) entry by entry
//
//   latent_heads   for prompts that bring all their keys along: per (token, head) the query [q_flat, rot(q_rot), 0 ...],
//                  the expanded key [U_k[h] c, k_r, 0 ...] and the value [U_v[h] c, 0 ...], all `hw` wide, for the
//                  ordinary attention kernels (whose heads then are this mixer's heads); latent_expand without a
//                  matrix then only gates and narrows the result
//
// Rotation: of the r rotated entries the first `rot_dims` are turned by the angle pos * rate_i (tables of cosines and
// sines per position come ready-made), in neighbouring pairs (2i, 2i+1) if `paired`, else entry i with i + rot_dims/2.
// Norms, rotation and the per-head sums are float32.
#include "common.cuh"

__device__ __forceinline__ float rot_entry(const float* x, int i, int rot_dims, int paired, const float* cs,
                                           const float* sn) {
    if (i >= rot_dims) return x[i];
    const int half = rot_dims >> 1;
    if (paired) {
        const int p = i >> 1;
        return (i & 1) ? x[i] * cs[p] + x[i - 1] * sn[p] : x[i] * cs[p] - x[i + 1] * sn[p];
    }
    return i < half ? x[i] * cs[i] - x[i + half] * sn[i] : x[i] * cs[i - half] + x[i - half] * sn[i - half];
}

template <typename T>
__global__ void latent_rows_kernel(const float* __restrict__ proj, int ld, int off_q, int off_kv, int q_rank, int n, int r,
                                   int rp, const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims,
                                   int paired, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                   const int* __restrict__ new_lens, T* __restrict__ cq_out, T* __restrict__ row_out,
                                   T* __restrict__ pages, const int* __restrict__ block_table, int table_width,
                                   int page_tokens, int ring_pages) {
    extern __shared__ float sh[];          // [r] the raw rotated part
    __shared__ float red[32];
    const int t = blockIdx.x;
    pdl_wait();
    pdl_launch();
    const float* row = proj + (size_t)t * ld;
    const int pos = tok_pos[t], b = tok_seq[t];
    // the query latent (q_rank == 0: the queries are projected directly and there is none)
    float ss = 0.f, inv = 0.f;
    if (q_rank > 0) {
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss = fmaf(row[off_q + i], row[off_q + i], ss);
        ss = block_sum(ss, red);
        inv = 1.f / sqrtf(ss / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            cq_out[(size_t)t * q_rank + i] = from_f32<T>(row[off_q + i] * inv * wq[i]);
    }
    // the cache row
    ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(row[off_kv + i], row[off_kv + i], ss);
    ss = block_sum(ss, red);
    inv = 1.f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < r; i += blockDim.x) sh[i] = row[off_kv + n + i];
    __syncthreads();
    T* dst_page = nullptr;
    // in a ring (a window's cache) only the last ring_pages * page_tokens positions of a sequence are written
    if (pages && pos < new_lens[b] && (ring_pages <= 0 || pos >= new_lens[b] - ring_pages * page_tokens)) {
        const int lp = ring_pages > 0 ? (pos / page_tokens) % ring_pages : pos / page_tokens;
        const int page = block_table[(size_t)b * table_width + lp];
        dst_page = pages + ((size_t)page * page_tokens + (pos % page_tokens)) * rp;
    }
    T* dst_row = row_out ? row_out + (size_t)t * rp : nullptr;
    const float* cs = cos_t + (size_t)pos * (rot_dims >> 1);
    const float* sn = sin_t + (size_t)pos * (rot_dims >> 1);
    for (int i = threadIdx.x; i < rp; i += blockDim.x) {
        float v = 0.f;
        if (i < n) v = row[off_kv + i] * inv * wkv[i];
        else if (i < n + r) v = rot_entry(sh, i - n, rot_dims, paired, cs, sn);
        const T o = from_f32<T>(v);
        if (dst_page) dst_page[i] = o;
        if (dst_row) dst_row[i] = o;
    }
}

template <typename T>
__global__ void latent_query_kernel(const float* __restrict__ q, int ldq, int H, int d, int r, int n, int rp,
                                    const T* __restrict__ uk, const float* __restrict__ cos_t,
                                    const float* __restrict__ sin_t, int rot_dims, int paired,
                                    const int* __restrict__ tok_pos, T* __restrict__ out) {
    extern __shared__ float sh[];          // [d + r] this head's query
    const int t = blockIdx.x, h = blockIdx.y;
    pdl_wait();
    pdl_launch();
    const float* qr = q + (size_t)t * ldq + (size_t)h * (d + r);
    for (int i = threadIdx.x; i < d + r; i += blockDim.x) sh[i] = qr[i];
    __syncthreads();
    const int pos = tok_pos[t];
    const float* cs = cos_t + (size_t)pos * (rot_dims >> 1);
    const float* sn = sin_t + (size_t)pos * (rot_dims >> 1);
    T* o = out + ((size_t)t * H + h) * rp;
    const T* w = uk + (size_t)h * d * n;            // [d, n]: row k holds what flat key entry k takes of the latent
    for (int i = threadIdx.x; i < rp; i += blockDim.x) {
        float v = 0.f;
        if (i < n) {
            for (int k = 0; k < d; ++k) v = fmaf(sh[k], to_f32<T>(w[(size_t)k * n + i]), v);
        } else if (i < n + r) {
            v = rot_entry(sh + d, i - n, rot_dims, paired, cs, sn);
        }
        o[i] = from_f32<T>(v);
    }
}

// q float32 [T, H * (d + r)]; kfv float32 [T, ldk]: head h's flat key at column h * d, its value at off_v + h * e;
// rows [T, rp]: the cache rows, whose entries n .. n + r - 1 are the rotated key part.
template <typename T>
__global__ void latent_heads_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ kfv, int ldk, int off_v,
                                    const T* __restrict__ rows, int rp, int n, int H, int d, int r, int e, int hw,
                                    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims,
                                    int paired, const int* __restrict__ tok_pos, T* __restrict__ q_out,
                                    T* __restrict__ k_out, T* __restrict__ v_out) {
    extern __shared__ float sh[];          // [r] this head's rotated query part, raw
    const int t = blockIdx.x, h = blockIdx.y;
    pdl_wait();
    pdl_launch();
    const float* qr = q + (size_t)t * ldq + (size_t)h * (d + r);
    for (int i = threadIdx.x; i < r; i += blockDim.x) sh[i] = qr[d + i];
    __syncthreads();
    const int pos = tok_pos[t];
    const float* cs = cos_t + (size_t)pos * (rot_dims >> 1);
    const float* sn = sin_t + (size_t)pos * (rot_dims >> 1);
    const size_t o = ((size_t)t * H + h) * hw;
    const float* kr = kfv + (size_t)t * ldk + (size_t)h * d;
    const float* vr = kfv + (size_t)t * ldk + off_v + (size_t)h * e;
    const T* rr = rows + (size_t)t * rp + n;
    for (int i = threadIdx.x; i < hw; i += blockDim.x) {
        T qv = from_f32<T>(0.f), kv = qv;
        if (i < d) { qv = from_f32<T>(qr[i]); kv = from_f32<T>(kr[i]); }
        else if (i < d + r) { qv = from_f32<T>(rot_entry(sh, i - d, rot_dims, paired, cs, sn)); kv = rr[i - d]; }
        q_out[o + i] = qv;
        k_out[o + i] = kv;
        v_out[o + i] = i < e ? from_f32<T>(vr[i]) : from_f32<T>(0.f);
    }
}

template <typename T>
__global__ void latent_expand_kernel(const T* __restrict__ lat, int H, int n, int rp, int e, const T* __restrict__ uv,
                                     const float* __restrict__ gate, int ldg, T* __restrict__ out) {
    extern __shared__ float sh[];          // [n] the head's mean latent
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    pdl_wait();
    pdl_launch();
    const T* lr = lat + ((size_t)t * H + h) * rp;
    for (int i = threadIdx.x; i < n; i += blockDim.x) sh[i] = to_f32<T>(lr[i]);
    __syncthreads();
    if (!uv) {                             // nothing to expand: the head's first e entries, gated
        for (int j = threadIdx.x; j < e; j += blockDim.x) {
            const size_t c = (size_t)h * e + j;
            float acc = sh[j];
            if (gate) acc *= 1.f / (1.f + expf(-gate[(size_t)t * ldg + c]));
            out[(size_t)t * H * e + c] = from_f32<T>(acc);
        }
        return;
    }
    for (int j = warp; j < e; j += n_warps) {
        const T* w = uv + ((size_t)h * e + j) * n;
        float acc = 0.f;
        for (int i = lane; i < n; i += 32) acc = fmaf(to_f32<T>(w[i]), sh[i], acc);
        acc = warp_sum(acc);
        if (lane == 0) {
            const size_t c = (size_t)h * e + j;
            if (gate) acc *= 1.f / (1.f + expf(-gate[(size_t)t * ldg + c]));
            out[(size_t)t * H * e + c] = from_f32<T>(acc);
        }
    }
}

TQ_API int tq_latent_rows(const float* proj, int ld, int off_q, int off_kv, int q_rank, int n, int r, int rp,
                          const float* wq, const float* wkv, float eps, const float* cos_t, const float* sin_t,
                          int rot_dims, int paired, const int* tok_pos, const int* tok_seq, const int* new_lens,
                          void* cq_out, void* row_out, void* pages, const int* block_table, int table_width,
                          int page_tokens, int ring_pages, int dtype, int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!proj || !wkv || !cos_t || !sin_t || !tok_pos || !tok_seq || !new_lens || q_rank < 0 ||
        (q_rank > 0 && (!wq || !cq_out)) || n <= 0 ||
        r < 0 || rp < n + r || rot_dims < 0 || rot_dims > r || (rot_dims & 1) || (pages && (!block_table || page_tokens <= 0)))
        return (int)cudaErrorInvalidValue;
    const int threads = (n >= 512 || q_rank >= 512) ? 256 : 128;
    const size_t smem = (size_t)(r > 0 ? r : 1) * sizeof(float);
    if (dtype == TQ_F32)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, latent_rows_kernel<float>, dim3(n_tokens), dim3(threads), smem, stream,
                             proj, ld, off_q, off_kv, q_rank, n, r, rp, wq, wkv, eps, cos_t, sin_t, rot_dims, paired,
                             tok_pos, tok_seq, new_lens, (float*)cq_out, (float*)row_out, (float*)pages, block_table,
                             table_width, page_tokens, ring_pages);
    if (dtype == TQ_BF16)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, latent_rows_kernel<bf16>, dim3(n_tokens), dim3(threads), smem, stream,
                             proj, ld, off_q, off_kv, q_rank, n, r, rp, wq, wkv, eps, cos_t, sin_t, rot_dims, paired,
                             tok_pos, tok_seq, new_lens, (bf16*)cq_out, (bf16*)row_out, (bf16*)pages, block_table,
                             table_width, page_tokens, ring_pages);
    return (int)cudaErrorInvalidValue;
}

TQ_API int tq_latent_query(const float* q, int ldq, int H, int d, int r, int n, int rp, const void* uk, const float* cos_t,
                           const float* sin_t, int rot_dims, int paired, const int* tok_pos, void* out, int dtype,
                           int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!q || !uk || !cos_t || !sin_t || !tok_pos || !out || H <= 0 || H > 65535 || d <= 0 || r < 0 || n <= 0 ||
        rp < n + r || rot_dims < 0 || rot_dims > r || (rot_dims & 1))
        return (int)cudaErrorInvalidValue;
    const int threads = rp > 128 ? 256 : 128;
    const size_t smem = (size_t)(d + r) * sizeof(float);
    const dim3 grid(n_tokens, H);
    if (dtype == TQ_F32)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, latent_query_kernel<float>, grid, dim3(threads), smem, stream, q, ldq, H, d, r,
                             n, rp, (const float*)uk, cos_t, sin_t, rot_dims, paired, tok_pos, (float*)out);
    if (dtype == TQ_BF16)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, latent_query_kernel<bf16>, grid, dim3(threads), smem, stream, q, ldq, H, d, r,
                             n, rp, (const bf16*)uk, cos_t, sin_t, rot_dims, paired, tok_pos, (bf16*)out);
    return (int)cudaErrorInvalidValue;
}

TQ_API int tq_latent_expand(const void* lat, int H, int n, int rp, int e, const void* uv, const float* gate, int ldg,
                            void* out, int dtype, int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!lat || !out || H <= 0 || H > 65535 || n <= 0 || rp < n || e <= 0 || (!uv && e > n)) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)n * sizeof(float);
    const dim3 grid(n_tokens, H);
    if (dtype == TQ_F32)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, latent_expand_kernel<float>, grid, dim3(128), smem, stream,
                             (const float*)lat, H, n, rp, e, (const float*)uv, gate, ldg, (float*)out);
    if (dtype == TQ_BF16)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, latent_expand_kernel<bf16>, grid, dim3(128), smem, stream,
                             (const bf16*)lat, H, n, rp, e, (const bf16*)uv, gate, ldg, (bf16*)out);
    return (int)cudaErrorInvalidValue;
}

TQ_API int tq_latent_heads(const float* q, int ldq, const float* kfv, int ldk, int off_v, const void* rows, int rp, int n, int H,
                           int d, int r, int e, int hw, const float* cos_t, const float* sin_t, int rot_dims, int paired,
                           const int* tok_pos, void* q_out, void* k_out, void* v_out, int dtype, int n_tokens,
                           cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!q || !kfv || !rows || !cos_t || !sin_t || !tok_pos || !q_out || !k_out || !v_out || H <= 0 || H > 65535 ||
        d <= 0 || r < 0 || e <= 0 || hw < d + r || hw < e || rp < n + r || rot_dims < 0 || rot_dims > r || (rot_dims & 1))
        return (int)cudaErrorInvalidValue;
    const dim3 grid(n_tokens, H);
    const size_t smem = (size_t)(r > 0 ? r : 1) * sizeof(float);
    if (dtype == TQ_F32)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, latent_heads_kernel<float>, grid, dim3(128), smem, stream, q, ldq, kfv, ldk,
                             off_v, (const float*)rows, rp, n, H, d, r, e, hw, cos_t, sin_t, rot_dims, paired, tok_pos,
                             (float*)q_out, (float*)k_out, (float*)v_out);
    if (dtype == TQ_BF16)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, latent_heads_kernel<bf16>, grid, dim3(128), smem, stream, q, ldq, kfv, ldk,
                             off_v, (const bf16*)rows, rp, n, H, d, r, e, hw, cos_t, sin_t, rot_dims, paired, tok_pos,
                             (bf16*)q_out, (bf16*)k_out, (bf16*)v_out);
    return (int)cudaErrorInvalidValue;
}
