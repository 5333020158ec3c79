// Routed experts: each token's feed-forward is a weighted sum of a few small gated feed-forwards
// chosen by a router.
//
//   moe_route     per token: logits z = W_r h in float; score s = sigmoid(z) (or a softmax over the
//                 experts); the `top` experts with the largest s + bias are chosen (the bias steers the
//                 choice only), ties to the lower index; the weights are the chosen s, optionally
//                 renormalised to sum 1
//   moe_gate_up   per (token, choice): act(W_gate[e] h) * (W_up[e] h), one warp per feature
//   moe_down      per token: sum over its choices, in order of choice, of weight * W_down[e] a
//
// The last two read an expert's matrices once per token that chose it: the right shape for decode
// steps, where tokens are few and the matrices stream from memory.  All sums are float and depend only
// on the token itself.
#include "common.cuh"

__device__ __forceinline__ float moe_act(float g, int act) {
    if (act == 1) return fmaxf(g, 0.0f);
    if (act == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.0f + expf(-g));
}

template <typename T, typename TW>
__global__ void __launch_bounds__(128) moe_route_kernel(const T* __restrict__ h, long h_ld, const TW* __restrict__ w_router,
                                                        const TW* __restrict__ bias, int* __restrict__ chosen,
                                                        float* __restrict__ weights, int width, int experts, int top,
                                                        int softmax_scores, int renormalise) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float route_s[];                  // [experts] scores, [experts] scores + bias
    float* score = route_s;
    float* pick = route_s + experts;
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* x = h + (long)t * h_ld;
    for (int e = warp; e < experts; e += 4) {
        const TW* wr = w_router + (long)e * width;
        float z = 0.0f;
        for (int i = lane; i < width; i += 32) z += to_f32<T>(x[i]) * to_f32<TW>(wr[i]);
        z = warp_sum(z);
        if (lane == 0) score[e] = z;
    }
    __syncthreads();
    if (warp != 0) return;
    if (softmax_scores) {
        float mx = -CUDART_INF_F;
        for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, score[e]);
        mx = warp_max(mx);
        float sum = 0.0f;
        for (int e = lane; e < experts; e += 32) sum += expf(score[e] - mx);
        sum = warp_sum(sum);
        for (int e = lane; e < experts; e += 32) score[e] = expf(score[e] - mx) / sum;
    } else {
        for (int e = lane; e < experts; e += 32) score[e] = 1.0f / (1.0f + expf(-score[e]));
    }
    for (int e = lane; e < experts; e += 32) pick[e] = score[e] + (bias ? to_f32<TW>(bias[e]) : 0.0f);
    __syncwarp();
    float total = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -CUDART_INF_F;
        int at = experts;
        for (int e = lane; e < experts; e += 32)
            if (pick[e] > best) { best = pick[e]; at = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= experts) at = 0;                      // every remaining score is NaN or -inf
        if (lane == 0) {
            chosen[(long)t * top + k] = at;
            weights[(long)t * top + k] = score[at];
            pick[at] = -CUDART_INF_F;
        }
        total += score[at];
        __syncwarp();
    }
    if (renormalise && lane == 0)
        for (int k = 0; k < top; ++k) weights[(long)t * top + k] /= total;
}

// w_gu: [experts][2 ff][width] (gate rows, then up rows); a: [tokens x top][ff] float
template <typename T, typename TW>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(const T* __restrict__ h, long h_ld, const TW* __restrict__ w_gu,
                                                          const int* __restrict__ chosen, float* __restrict__ a,
                                                          int width, int ff, int top, int act) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float moe_x[];                    // [width]
    const int pair = blockIdx.x, t = pair / top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < width; i += blockDim.x) moe_x[i] = to_f32<T>(h[(long)t * h_ld + i]);
    __syncthreads();
    const int f = blockIdx.y * 8 + warp;
    if (f >= ff) return;
    const TW* wg = w_gu + ((long)chosen[pair] * 2 * ff + f) * width;
    const TW* wu = wg + (long)ff * width;
    float g = 0.0f, u = 0.0f;
    for (int i = lane; i < width; i += 32) {
        g += moe_x[i] * to_f32<TW>(wg[i]);
        u += moe_x[i] * to_f32<TW>(wu[i]);
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) a[(long)pair * ff + f] = moe_act(g, act) * u;
}

// w_down: [experts][width][ff]
template <typename T, typename TW>
__global__ void __launch_bounds__(256) moe_down_kernel(const float* __restrict__ a, const TW* __restrict__ w_down,
                                                       const int* __restrict__ chosen, const float* __restrict__ weights,
                                                       T* __restrict__ out, long out_ld, int width, int ff, int top) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.y * 8 + warp;
    if (c >= width) return;
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) {
        const long pair = (long)t * top + k;
        const TW* wd = w_down + ((long)chosen[pair] * width + c) * ff;
        const float* ar = a + pair * ff;
        float y = 0.0f;
        for (int i = lane; i < ff; i += 32) y += ar[i] * to_f32<TW>(wd[i]);
        sum += weights[pair] * warp_sum(y);
    }
    if (lane == 0) out[(long)t * out_ld + c] = from_f32<T>(sum);
}

FL_API int fl_moe_route(const void* h, int dtype, long h_ld, const void* w_router, const void* bias, int w_dtype,
                        int* chosen, float* weights, int n_tokens, int width, int experts, int top, int softmax_scores,
                        int renormalise, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top < 1 || top > experts || (size_t)experts * 8 > 48 * 1024) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(dtype, T, FL_DISPATCH(w_dtype, TW,
        return fl_launch(moe_route_kernel<T, TW>, dim3(n_tokens), dim3(128), (size_t)experts * 2 * sizeof(float), stream,
                         (const T*)h, h_ld, (const TW*)w_router, (const TW*)bias, chosen, weights, width, experts, top,
                         softmax_scores, renormalise)));
    return 0;
}

FL_API int fl_moe_experts(const void* h, int dtype, long h_ld, const void* w_gu, const void* w_down, int w_dtype,
                          const int* chosen, const float* weights, float* a, void* out, long out_ld, int n_tokens,
                          int width, int ff, int top, int act, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if ((size_t)width * sizeof(float) > 48 * 1024 || (ff + 7) / 8 > 65535 || (width + 7) / 8 > 65535 || act < 0 || act > 2)
        return (int)cudaErrorInvalidValue;
    int rc = 0;
    FL_DISPATCH(dtype, T, FL_DISPATCH(w_dtype, TW,
        rc = fl_launch(moe_gate_up_kernel<T, TW>, dim3(n_tokens * top, (ff + 7) / 8), dim3(256),
                       (size_t)width * sizeof(float), stream, (const T*)h, h_ld, (const TW*)w_gu, chosen, a, width, ff,
                       top, act)));
    if (rc) return rc;
    FL_DISPATCH(dtype, T, FL_DISPATCH(w_dtype, TW,
        return fl_launch(moe_down_kernel<T, TW>, dim3(n_tokens, (width + 7) / 8), dim3(256), 0, stream, (const float*)a,
                         (const TW*)w_down, chosen, weights, (T*)out, out_ld, width, ff, top)));
    return 0;
}
