// A matrix memory with exponential gates (the mLSTM of xLSTM), the two kernels around the scan of
// linear_scan.cu.  Per head and token, with raw gate values i~ and f~ (projection plus bias):
//
//   i = cap * tanh(i~ / cap)                      log of the input gate
//   f = logsigmoid(cap * tanh(f~ / cap))          log of the forget gate
//   m_t = max(f + m_{t-1}, i)                     a running maximum, m_0 = 0, that keeps the exponentials in range
//   S_t = exp(f + m_{t-1} - m_t) S_{t-1} + exp(i - m_t) k v^T          (d x e)
//   n_t = exp(f + m_{t-1} - m_t) n_{t-1} + exp(i - m_t) k              (d)
//   o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + floor)
//
// n rides in S as one more value column whose v entry is 1, so the update is the scan with one decay per head and
// token (SCAN_GATED: decay a_t = exp(f + m_{t-1} - m_t), step size b_t = exp(i - m_t)) over values of e + 1 columns,
// padded to a multiple of four; column e of its result is n_t . q.
//
//   mlstm_gates    a warp per (sequence, head) walks the sequence's tokens of the step: the lanes take 32 tokens'
//                  gates at a time (tanh, logsigmoid: off the chain), the chain m_t = max(f + m, i) runs over
//                  shuffled values (an add and a max per token), then each lane forms its token's a, b and m;
//                  m is read from and written back to the sequence's state
//   mlstm_read     a warp per (token, head): the division above, the head's RMS norm (x / sqrt(mean(x^2) + eps)),
//                  the norm's weight and the sigmoid output gate
// Everything here is float32; only mlstm_read's result is rounded to the activations' type.
#include "common.cuh"

__device__ __forceinline__ float log_sigmoid(float z) {
    // -log(1 + exp(-z)), without overflow on either side
    return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z));
}

__global__ void __launch_bounds__(128)
mlstm_gates_kernel(const float* __restrict__ in_raw, const float* __restrict__ f_raw, int ld, float cap,
                   const int* __restrict__ cu_seqlens, const int* __restrict__ slots, float* __restrict__ state_m,
                   long long state_stride, int H, float* __restrict__ scal, int n_seqs) {
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= n_seqs * H) return;
    const int b = w / H, h = w - b * H;
    pdl_wait();
    pdl_launch();
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    float* mp = state_m + (size_t)slots[b] * state_stride + h;
    float m = *mp;
    // the raw gates of the chunk after this one are asked for before the chain of this one runs
    float in_next = 0.f, f_next = 0.f;
    if (t0 + lane < t1) {
        in_next = in_raw[(size_t)(t0 + lane) * ld + h];
        f_next = f_raw[(size_t)(t0 + lane) * ld + h];
    }
    for (int base = t0; base < t1; base += 32) {
        const int t = base + lane;
        const bool valid = t < t1;
        const float in_now = in_next, f_now = f_next;
        if (t + 32 < t1) {
            in_next = in_raw[(size_t)(t + 32) * ld + h];
            f_next = f_raw[(size_t)(t + 32) * ld + h];
        }
        // a lane past the sequence's end carries the gates that leave m as it is: f = 0, i = -inf
        float ig = -INFINITY, fg = 0.f;
        if (valid) {
            ig = cap * tanhf(in_now / cap);
            fg = log_sigmoid(cap * tanhf(f_now / cap));
        }
        float m_before = 0.f, m_mine = 0.f;
#pragma unroll
        for (int s = 0; s < 32; ++s) {                        // (the shuffles do not wait for the chain: only add and max do)
            const float fi = __shfl_sync(0xffffffffu, ig, s);
            const float ff = __shfl_sync(0xffffffffu, fg, s);
            const float m_new = fmaxf(ff + m, fi);
            if (lane == s) { m_before = m; m_mine = m_new; }
            m = m_new;
        }
        if (valid) {
            float4 o;
            o.x = expf(fg + m_before - m_mine);
            o.y = expf(ig - m_mine);
            o.z = m_mine;
            o.w = 0.f;
            reinterpret_cast<float4*>(scal)[(size_t)t * H + h] = o;
        }
    }
    if (lane == 0) *mp = m;
}

// in_raw / f_raw: column slices (row stride ld) of the projected float32 rows, one entry per head; scal [T, H, 4]
// receives (a, b, m, 0); state_m points at the heads' m of slot 0, slots are state_stride floats apart.
TQ_API int tq_mlstm_gates(const float* in_raw, const float* f_raw, int ld, float cap, const int* cu_seqlens,
                          const int* slots, float* state_m, long long state_stride, int H, float* scal, int n_seqs,
                          cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (!in_raw || !f_raw || !cu_seqlens || !slots || !state_m || !scal || H <= 0 || !(cap > 0.f) ||
        (reinterpret_cast<uintptr_t>(scal) & 15))
        return (int)cudaErrorInvalidValue;
    const int warps = n_seqs * H;
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, mlstm_gates_kernel, dim3((warps + 3) / 4), dim3(128), 0, stream, in_raw,
                         f_raw, ld, cap, cu_seqlens, slots, state_m, state_stride, H, scal, n_seqs);
}

#define MR_MAX_PER_LANE 16      // value widths up to 512

template <typename TO>
__global__ void __launch_bounds__(128)
mlstm_read_kernel(const float* __restrict__ o, int ea, int e, const float* __restrict__ scal,
                  const float* __restrict__ gate, int ldg, const float* __restrict__ norm_w, float q_scale, float floor_,
                  float eps, int H, TO* __restrict__ out, int n_pairs) {
    const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (p >= n_pairs) return;
    const int t = p / H, h = p - t * H;
    pdl_wait();
    pdl_launch();
    const float* row = o + (size_t)p * ea;
    // every load of the warp is asked for at once: the values, their gates, n . q and m
    float v[MR_MAX_PER_LANE], g[MR_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MR_MAX_PER_LANE; ++i) {
        const int j = lane + 32 * i;
        v[i] = j < e ? row[j] : 0.f;
        g[i] = j < e ? gate[(size_t)t * ldg + h * e + j] : 0.f;
    }
    const float nq = row[e];
    const float m = scal[(size_t)p * 4 + 2];
    const float den = fmaxf(fabsf(nq * q_scale), expf(-m)) + floor_;
    const float by_den = q_scale / den;               // one division per (token, head)
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MR_MAX_PER_LANE; ++i) {
        v[i] *= by_den;
        ss = fmaf(v[i], v[i], ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)e + eps);
#pragma unroll
    for (int i = 0; i < MR_MAX_PER_LANE; ++i) {
        const int j = lane + 32 * i;
        if (j < e) {
            const int c = h * e + j;
            // (a bfloat16 result keeps 8 bits: the fast exponential and division do)
            const float sg = sizeof(TO) == 2 ? __fdividef(1.f, 1.f + __expf(-g[i])) : 1.f / (1.f + expf(-g[i]));
            out[(size_t)t * H * e + c] = from_f32<TO>(v[i] * inv * norm_w[c] * sg);
        }
    }
}

// o [T, H * ea] float32: the scan's result, per head e value columns, then n . q, then padding; scal [T, H, 4] as
// mlstm_gates left it; gate: float32 rows (stride ldg) of H * e gate values before the sigmoid; norm_w [H * e];
// out [T, H * e] float32 or bfloat16.  q_scale: the factor the queries were NOT multiplied with before the scan.
TQ_API int tq_mlstm_read(const float* o, int ea, int e, const float* scal, const float* gate, int ldg,
                         const float* norm_w, float q_scale, float floor_, float eps, int H, void* out, int out_dtype,
                         int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!o || !scal || !gate || !norm_w || !out || e <= 0 || e > 32 * MR_MAX_PER_LANE || ea <= e || H <= 0)
        return (int)cudaErrorInvalidValue;
    const int n_pairs = n_tokens * H;
    const dim3 grid((n_pairs + 3) / 4);
    if (out_dtype == TQ_F32)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, mlstm_read_kernel<float>, grid, dim3(128), 0, stream, o, ea, e, scal, gate,
                             ldg, norm_w, q_scale, floor_, eps, H, (float*)out, n_pairs);
    if (out_dtype == TQ_BF16)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, mlstm_read_kernel<bf16>, grid, dim3(128), 0, stream, o, ea, e, scal, gate,
                             ldg, norm_w, q_scale, floor_, eps, H, (bf16*)out, n_pairs);
    return (int)cudaErrorInvalidValue;
}
