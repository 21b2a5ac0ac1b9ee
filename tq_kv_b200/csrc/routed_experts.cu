// A feed-forward of many small experts of which each token uses a few, named by
// a table (or any int32 list): expert e is  W_down[e] (silu(W_gate[e] x) * (W_up[e] x)),
// and a token's result is the mean of its experts' results, or their sum with a weight per (token, expert)
// where a router gives weights (router_choice below).
//
// The experts' weights are stacked: w_gu [E, 2*F, W] (an expert's gate rows, then its up rows) and
// w_down [E, W, F].  choice [T, top] int32 names each token's experts.
//
// Few tokens (decoding), and the float32 path: every (token, expert) pair is a row-times-matrix product of
// its own, a warp per output entry, 16-byte loads, float32 sums.
//   routed_gate_up:  act[t*top + s, i] = silu(x[t] . gate[e][i]) * (x[t] . up[e][i])
//   routed_down:     y[t, c] (+)= 1/top * sum_s act[t*top + s] . down[e_s][c]     (the experts in the table's order)
// Many tokens: the rows are sorted by expert so that each expert's rows form whole tiles of a matrix product
// (routed_plan / routed_gather / routed_combine below; the products themselves are csrc/gemm_tc.cu's).
#include "common.cuh"

// ---- choice: experts of each token from a table indexed by the token id ------------------------------------------
__global__ void table_choice_kernel(const int* __restrict__ tokens, const int* __restrict__ table, int vocab, int top,
                                    int n_experts, int* __restrict__ choice, int n) {
    pdl_wait();
    pdl_launch();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int t = i / top, s = i - t * top;
    int tok = tokens[t];
    if (tok < 0 || tok >= vocab) tok = 0;                 // (the host has checked the ids)
    int e = table[(size_t)tok * top + s];
    if (e < 0 || e >= n_experts) e = 0;                   // (checked when the table is bound)
    choice[i] = e;
}

TQ_API int tq_table_choice(const int* tokens, const int* table, int vocab, int top, int n_experts, int* choice,
                           int n_tokens, cudaStream_t stream) {
    const int n = n_tokens * top;
    if (n <= 0) return 0;
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, table_choice_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tokens,
                         table, vocab, top, n_experts, choice, n);
}

// ---- choice: experts of each token from a router's logits -------------------------------------------------------
// scores s = sigmoid(logit); the `top` largest are chosen (the lowest index first among equals); their weights
// are  scale * s / (sum of the chosen s + floor).  The choice compares the logits themselves: the sigmoid keeps
// their order, but in float32 it is 1 for every logit above 17 and would make equals of them.  A warp per token;
// float32 throughout.
__global__ void __launch_bounds__(128)
router_choice_kernel(const float* __restrict__ logits, int ld, int n_experts, int top, float scale, float floor_,
                     int* __restrict__ choice, float* __restrict__ weights, int n_tokens) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= n_tokens) return;
    pdl_wait();
    pdl_launch();
    const float* z = logits + (size_t)t * ld;
    float total = 0.f;
    for (int s = 0; s < top; ++s) {
        float best = 0.f;
        int best_e = n_experts;                           // n_experts: this lane has found none yet
        for (int e = lane; e < n_experts; e += 32) {
            bool taken = false;
            for (int r = 0; r < s; ++r) taken |= choice[t * top + r] == e;
            const float v = z[e];                        // the order of the logits is the order of the scores
            if (!taken && (best_e == n_experts || v > best)) { best = v; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (oe < n_experts && (best_e == n_experts || ob > best || (ob == best && oe < best_e))) { best = ob; best_e = oe; }
        }
        const float score = 1.f / (1.f + expf(-best));
        if (lane == 0) { choice[t * top + s] = best_e; weights[t * top + s] = score; }
        __syncwarp();
        total += score;
    }
    const float f = scale / (total + floor_);
    for (int s = lane; s < top; s += 32) weights[t * top + s] *= f;
}

TQ_API int tq_router_choice(const float* logits, int ld, int n_experts, int top, float scale, float floor_, int* choice,
                            float* weights, int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!logits || !choice || !weights || top < 1 || top > n_experts) return (int)cudaErrorInvalidValue;
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, router_choice_kernel, dim3((n_tokens + 3) / 4), dim3(128), 0, stream, logits,
                         ld, n_experts, top, scale, floor_, choice, weights, n_tokens);
}

// ---- a warp's inner product over n entries ---------------------------------------------------------------------
template <typename TA, typename TB>
__device__ __forceinline__ float warp_dot(const TA* __restrict__ a, const TB* __restrict__ b, int n, bool vec) {
    const int lane = threadIdx.x & 31;
    float acc = 0.f;
    if (vec) {                                            // n % 8 == 0, both rows 16-byte aligned
        for (int d = lane * 8; d < n; d += 256) {
            float av[8], bv[8];
            if constexpr (sizeof(TA) == 2) load16_f32<TA>(a + d, av);
            else { load16_f32<TA>(a + d, av); load16_f32<TA>(a + d + 4, av + 4); }
            if constexpr (sizeof(TB) == 2) load16_f32<TB>(b + d, bv);
            else { load16_f32<TB>(b + d, bv); load16_f32<TB>(b + d + 4, bv + 4); }
#pragma unroll
            for (int e = 0; e < 8; ++e) acc = fmaf(av[e], bv[e], acc);
        }
    } else {
        for (int d = lane; d < n; d += 32) acc = fmaf(to_f32<TA>(a[d]), to_f32<TB>(b[d]), acc);
    }
    return warp_sum(acc);
}

// grid (T*top, ceil(F / 8)), 8 warps: warp w computes entry i = blockIdx.y*8 + w
template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
routed_gate_up_kernel(const TX* __restrict__ x, int ldx, const TW* __restrict__ w_gu, const int* __restrict__ choice,
                      int top, int W, int F, TO* __restrict__ act, bool vec) {
    const int pair = blockIdx.x;
    const int i = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (i >= F) return;
    pdl_wait();
    pdl_launch();
    const int e = choice[pair];
    const TX* xr = x + (size_t)(pair / top) * ldx;
    const TW* wg = w_gu + ((size_t)e * 2 * F + i) * W;
    const float g = warp_dot<TX, TW>(xr, wg, W, vec);
    const float u = warp_dot<TX, TW>(xr, wg + (size_t)F * W, W, vec);
    if ((threadIdx.x & 31) == 0) act[(size_t)pair * F + i] = from_f32<TO>(g / (1.f + expf(-g)) * u);
}

// grid (T, ceil(W / 8)), 8 warps: warp w computes column c = blockIdx.y*8 + w
template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
routed_down_kernel(const TA* __restrict__ act, const TW* __restrict__ w_down, const int* __restrict__ choice,
                   const float* __restrict__ weights, int top, int W, int F, float* __restrict__ y, int accumulate,
                   bool vec) {
    const int t = blockIdx.x;
    const int c = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (c >= W) return;
    pdl_wait();
    pdl_launch();
    float sum = 0.f;
    for (int s = 0; s < top; ++s) {
        const int e = choice[t * top + s];
        const float part = warp_dot<TA, TW>(act + (size_t)(t * top + s) * F, w_down + ((size_t)e * W + c) * F, F, vec);
        sum = weights ? fmaf(weights[t * top + s], part, sum) : sum + part;
    }
    if ((threadIdx.x & 31) == 0) {
        float* o = y + (size_t)t * W + c;
        const float v = weights ? sum : sum / (float)top;
        *o = accumulate ? *o + v : v;
    }
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// x [T, W] (row stride ldx), act [T*top, F] of x's dtype (scratch), y [T, W] float32.  Weights float32 or bfloat16.
TQ_API int tq_routed_experts_rows(const void* x, int x_dtype, int ldx, const void* w_gu, const void* w_down, int w_dtype,
                                  const int* choice, const float* weights, int top, int n_tokens, int W, int F,
                                  void* act, float* y, int accumulate, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top < 1 || W <= 0 || F <= 0) return (int)cudaErrorInvalidValue;
    const int xs = x_dtype == TQ_BF16 ? 2 : 4, ws = w_dtype == TQ_BF16 ? 2 : 4;
    const bool vec_up = W % 8 == 0 && aligned16(x) && aligned16(w_gu) && ((size_t)ldx * xs) % 16 == 0;
    const bool vec_down = F % 8 == 0 && aligned16(act) && aligned16(w_down);
    (void)ws;
    const dim3 g1(n_tokens * top, (F + 7) / 8), g2(n_tokens, (W + 7) / 8);
    if (g1.y > 65535 || g2.y > 65535) return (int)cudaErrorInvalidValue;
    int st;
#define TQ_RUN(TX, TW)                                                                                                \
    st = tq_launch_pdl(TQ_PDL_ELEMENTWISE, routed_gate_up_kernel<TX, TW, TX>, g1, dim3(256), 0, stream, (const TX*)x, \
                       ldx, (const TW*)w_gu, choice, top, W, F, (TX*)act, vec_up);                                   \
    if (st) return st;                                                                                                \
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, routed_down_kernel<TX, TW>, g2, dim3(256), 0, stream, (const TX*)act,   \
                         (const TW*)w_down, choice, weights, top, W, F, y, accumulate, vec_down)
    if (x_dtype == TQ_F32 && w_dtype == TQ_F32) { TQ_RUN(float, float); }
    if (x_dtype == TQ_F32 && w_dtype == TQ_BF16) { TQ_RUN(float, bf16); }
    if (x_dtype == TQ_BF16 && w_dtype == TQ_BF16) { TQ_RUN(bf16, bf16); }
#undef TQ_RUN
    return (int)cudaErrorInvalidValue;
}

// ---- many tokens: rows sorted by expert ---------------------------------------------------------------------------
// One block plans the step: it counts the (token, expert) pairs of each expert, gives each expert a run of whole
// tiles of `tile` rows in a sorted buffer (experts in index order), tells every tile which rows of the stacked
// weights it multiplies with (tile_b_up / tile_b_down: the expert's first row there; -1 for tiles past the last
// used one) and gives each pair its row in the buffer (pos).  Which of an expert's rows a pair gets depends on
// the order the threads arrive in; a row's result does not depend on where in a tile it lies.
__global__ void __launch_bounds__(1024)
routed_plan_kernel(const int* __restrict__ choice, int n_pairs, int n_experts, int tile, int up_rows, int down_rows,
                   int max_tiles, int* __restrict__ pos, int* __restrict__ tile_b_up, int* __restrict__ tile_b_down) {
    extern __shared__ int plan_sh[];         // counts [E], first row [E], cursor [E]
    int* counts = plan_sh;
    int* first = plan_sh + n_experts;
    int* cursor = plan_sh + 2 * n_experts;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
    pdl_wait();
    pdl_launch();
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&counts[choice[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int e = 0; e < n_experts; ++e) {
            first[e] = t * tile;
            const int n = (counts[e] + tile - 1) / tile;
            for (int i = 0; i < n && t < max_tiles; ++i, ++t) {
                tile_b_up[t] = e * up_rows;
                tile_b_down[t] = e * down_rows;
            }
        }
        for (; t < max_tiles; ++t) { tile_b_up[t] = -1; tile_b_down[t] = -1; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = choice[i];
        pos[i] = first[e] + atomicAdd(&cursor[e], 1);
    }
}

// sorted[pos[i]] = x[i / top]: a warp per pair, 16-byte copies (W % 8 == 0, bfloat16)
__global__ void __launch_bounds__(256)
routed_gather_kernel(const bf16* __restrict__ x, int ldx, const int* __restrict__ pos, int top, int W, int n_pairs,
                     bf16* __restrict__ sorted) {
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= n_pairs) return;
    pdl_wait();
    pdl_launch();
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(i / top) * ldx);
    uint4* dst = reinterpret_cast<uint4*>(sorted + (size_t)pos[i] * W);
    for (int d = lane; d < W / 8; d += 32) dst[d] = src[d];
}

// y[t] (=, +=) 1/top * sum_s out[pos[t*top + s]] (the experts in the table's order): float32, W % 4 == 0
__global__ void __launch_bounds__(256)
routed_combine_kernel(const float* __restrict__ out, const int* __restrict__ pos, const float* __restrict__ weights,
                      int top, int W, int n_tokens, float* __restrict__ y, int accumulate) {
    pdl_wait();
    pdl_launch();
    const int per_row = W / 4;
    const float inv = weights ? 1.f : 1.f / (float)top;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < (size_t)n_tokens * per_row;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / per_row), c = (int)(idx - (size_t)t * per_row);
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < top; ++s) {
            const float4 v = reinterpret_cast<const float4*>(out + (size_t)pos[t * top + s] * W)[c];
            const float ws = weights ? weights[t * top + s] : 1.f;
            a.x = fmaf(ws, v.x, a.x); a.y = fmaf(ws, v.y, a.y); a.z = fmaf(ws, v.z, a.z); a.w = fmaf(ws, v.w, a.w);
        }
        float4* o = reinterpret_cast<float4*>(y + (size_t)t * W) + c;
        if (accumulate) {
            const float4 old = *o;
            *o = make_float4(old.x + a.x * inv, old.y + a.y * inv, old.z + a.z * inv, old.w + a.w * inv);
        } else {
            *o = make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
        }
    }
}

// The plan and the gather of a step.  choice [T*top]; pos [T*top], tile_b_up / tile_b_down [max_tiles] (outputs);
// sorted [max_tiles*tile, W] bfloat16 (rows that no pair owns keep what they held: nobody reads their results).
TQ_API int tq_routed_sort(const void* x, int ldx, const int* choice, int top, int n_tokens, int W, int n_experts,
                          int tile, int up_rows, int down_rows, int max_tiles, int* pos, int* tile_b_up,
                          int* tile_b_down, void* sorted, cudaStream_t stream) {
    const int n_pairs = n_tokens * top;
    if (n_pairs <= 0) return 0;
    if (W % 8 || ldx % 8 || n_experts < 1 || n_experts > 4096 || tile < 1 || !aligned16(x) || !aligned16(sorted))
        return (int)cudaErrorInvalidValue;
    if (max_tiles < (n_pairs + tile - 1) / tile + n_experts - 1 && max_tiles < n_pairs) return (int)cudaErrorInvalidValue;
    int st = tq_launch_pdl(TQ_PDL_ELEMENTWISE, routed_plan_kernel, dim3(1), dim3(1024), (size_t)3 * n_experts * sizeof(int),
                           stream, choice, n_pairs, n_experts, tile, up_rows, down_rows, max_tiles, pos, tile_b_up,
                           tile_b_down);
    if (st) return st;
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, routed_gather_kernel, dim3((n_pairs + 7) / 8), dim3(256), 0, stream,
                         (const bf16*)x, ldx, (const int*)pos, top, W, n_pairs, (bf16*)sorted);
}

TQ_API int tq_routed_combine(const float* out, const int* pos, const float* weights, int top, int n_tokens, int W,
                             float* y, int accumulate, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (W % 4 || !aligned16(out) || !aligned16(y)) return (int)cudaErrorInvalidValue;
    size_t blocks = ((size_t)n_tokens * (W / 4) + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, routed_combine_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, out, pos,
                         weights, top, W, n_tokens, y, accumulate);
}
