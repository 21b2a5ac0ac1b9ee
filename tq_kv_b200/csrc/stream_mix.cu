// A residual stream kept as S parallel streams (hyper-connections).
//
// The streams are one float32 tensor xs [S, T, W], stream-major.  A sublayer
// reads the combination u = sum_s read[s] * xs[s], works on norm(u), and its
// result y enters all streams at once:
//     xs_new[r] = sum_s mix[s, r] * xs[s] + write[r] * y        (mix is indexed [from, to]).
// One kernel does both ends of a sublayer boundary for a token: it applies the
// write of the sublayer that has just finished (if any) and prepares the input
// of the next reader (if any): u, and optionally its RMS norm
// u / sqrt(mean(u^2) + eps) * w, in the dtype the reader wants.  So a layer of
// two sublayers costs two launches, and the sum of the streams that the final
// norm reads is the same kernel with read = 1.  All sums are float32.
#include "common.cuh"

#define SM_MAX_STREAMS 8

struct StreamCoefs {
    float mix[SM_MAX_STREAMS * SM_MAX_STREAMS];
    float write[SM_MAX_STREAMS];
    float read[SM_MAX_STREAMS];
};

// grid: one block per row r (token rows[r], or r).  y/mix/write may be null (no write), read may be null
// (no output).  u is held in shared memory [W] between the sum of squares and the scaling.
// NS: the number of streams where the kernel is built for exactly that many (1 to 4: the streams' values of a
// thread stay in few registers and three or four blocks share an SM), or SM_MAX_STREAMS for any number up to that.
template <typename TO, int VEC, int NS>
__global__ void __launch_bounds__(256, NS <= 3 ? 4 : (NS == 4 ? 3 : 1))
streams_step_kernel(float* __restrict__ xs, int S_any, int T, int W, const float* __restrict__ y,
                    const float* __restrict__ mix, const float* __restrict__ write, const float* __restrict__ read,
                    const float* __restrict__ norm_w, float eps, TO* __restrict__ out,
                    const int* __restrict__ rows) {
    const int S = NS < SM_MAX_STREAMS ? NS : S_any;
    extern __shared__ float u_sh[];
    __shared__ float red[32];
    __shared__ StreamCoefs cf;
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    // the coefficients are weights: they do not depend on the kernel before
    if (threadIdx.x < S * S && mix) cf.mix[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < S) {
        cf.write[threadIdx.x] = write ? write[threadIdx.x] : 0.f;
        cf.read[threadIdx.x] = read ? read[threadIdx.x] : 0.f;
    }
    pdl_wait();
    pdl_launch();
    __syncthreads();
    const size_t stride = (size_t)T * W;
    float* row = xs + (size_t)t * W;
    float ss = 0.f;
    for (int i = threadIdx.x * VEC; i < W; i += blockDim.x * VEC) {
        float x[NS][VEC];
#pragma unroll
        for (int s = 0; s < NS; ++s)
            if (s < S) {
                if constexpr (VEC == 4) {
                    const float4 v = *reinterpret_cast<const float4*>(row + s * stride + i);
                    x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3] = v.w;
                } else {
                    x[s][0] = row[s * stride + i];
                }
            }
        if (y) {
            float yv[VEC];
            if constexpr (VEC == 4) {
                const float4 v = *reinterpret_cast<const float4*>(y + (size_t)t * W + i);
                yv[0] = v.x; yv[1] = v.y; yv[2] = v.z; yv[3] = v.w;
            } else {
                yv[0] = y[(size_t)t * W + i];
            }
            float nx[NS][VEC];
#pragma unroll
            for (int to = 0; to < NS; ++to)
                if (to < S) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        float a = cf.write[to] * yv[e];
#pragma unroll
                        for (int s = 0; s < NS; ++s)
                            if (s < S) a = fmaf(cf.mix[s * S + to], x[s][e], a);
                        nx[to][e] = a;
                    }
                }
#pragma unroll
            for (int s = 0; s < NS; ++s)
                if (s < S) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) x[s][e] = nx[s][e];
                    if (rows) continue;          // a selection of rows only reads: the streams stay as they were
                    if constexpr (VEC == 4)
                        *reinterpret_cast<float4*>(row + s * stride + i) =
                            make_float4(x[s][0], x[s][1], x[s][2], x[s][3]);
                    else
                        row[s * stride + i] = x[s][0];
                }
        }
        if (out) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                float u = 0.f;
#pragma unroll
                for (int s = 0; s < NS; ++s)
                    if (s < S) u = fmaf(cf.read[s], x[s][e], u);
                u_sh[i + e] = u;
                ss = fmaf(u, u, ss);
            }
        }
    }
    if (!out) return;
    float inv = 1.f;
    if (norm_w) inv = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
    // (each thread reads back only what it wrote itself)
    TO* o = out + (size_t)r * W;
    for (int i = threadIdx.x * VEC; i < W; i += blockDim.x * VEC) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const float u = u_sh[i + e];
            o[i + e] = from_f32<TO>(norm_w ? u * inv * norm_w[i + e] : u);
        }
    }
}

// xs: [S, T, W] float32.  y: [T, W] float32 or null.  mix [S, S], write [S], read [S], norm_w [W]: float32 or
// null.  out: [n_rows, W] of out_dtype or null.  rows: int32 [n_rows] or null (then n_rows == T); with rows
// given the streams are not changed: the write is applied on the way to `out` only.
TQ_API int tq_streams_step(float* xs, int S, int T, int W, const float* y, const float* mix, const float* write,
                           const float* read, const float* norm_w, float eps, void* out, int out_dtype,
                           const int* rows, int n_rows, cudaStream_t stream) {
    if (n_rows <= 0 || T <= 0) return 0;
    if (S < 1 || S > SM_MAX_STREAMS || W <= 0 || W > 12288) return (int)cudaErrorInvalidValue;
    if (y && (!mix || !write)) return (int)cudaErrorInvalidValue;
    if (out && !read) return (int)cudaErrorInvalidValue;
    if (!y && !out) return 0;
    const size_t smem = out ? (size_t)W * sizeof(float) : 0;
    const bool vec = (W % 4 == 0) && ((reinterpret_cast<uintptr_t>(xs) | reinterpret_cast<uintptr_t>(y)) % 16 == 0);
#define TQ_LAUNCH_NS(TO, V, NS)                                                                                  \
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, streams_step_kernel<TO, V, NS>, dim3(n_rows), dim3(256), smem,      \
                         stream, xs, S, T, W, y, mix, write, read, norm_w, eps, (TO*)out, rows)
#define TQ_LAUNCH(TO, V)                                                                                         \
    switch (S) {                                                                                                 \
        case 1: TQ_LAUNCH_NS(TO, V, 1);                                                                          \
        case 2: TQ_LAUNCH_NS(TO, V, 2);                                                                          \
        case 3: TQ_LAUNCH_NS(TO, V, 3);                                                                          \
        case 4: TQ_LAUNCH_NS(TO, V, 4);                                                                          \
        default: TQ_LAUNCH_NS(TO, V, SM_MAX_STREAMS);                                                            \
    }
    if (out_dtype == TQ_F32 || !out) {
        if (vec) TQ_LAUNCH(float, 4)
        TQ_LAUNCH(float, 1)
    }
    if (out_dtype == TQ_BF16) {
        if (vec) TQ_LAUNCH(bf16, 4)
        TQ_LAUNCH(bf16, 1)
    }
#undef TQ_LAUNCH
#undef TQ_LAUNCH_NS
    return (int)cudaErrorInvalidValue;
}

// xs[s] = x for every stream s.
__global__ void streams_fill_kernel(const float* __restrict__ x, float* __restrict__ xs, int S, size_t n) {
    pdl_wait();
    pdl_launch();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        for (int s = 0; s < S; ++s) xs[(size_t)s * n + i] = v;
    }
}

TQ_API int tq_streams_fill(const float* x, float* xs, int S, size_t n, cudaStream_t stream) {
    if (n == 0 || S <= 0) return 0;
    size_t blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, streams_fill_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, xs, S, n);
}
