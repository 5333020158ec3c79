// Gated delta rule: a linear-attention mixer whose memory is one matrix per head.
//
// Per head, with a state S [dim x vdim] in float that a request carries from token to token:
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// where q, k (unit vectors per head, q times `q_scale`) and v come from projections that pass a short
// causal convolution over time and silu; beta = sigmoid(b) and g = exp(-exp(A_log) softplus(a + dt_bias))
// are per head and token.  The read-out sees the token's own write.
//
// Four kernels, all float inside:
//   delta_prep        per token and head: convolution over the last `taps` inputs (from the step's rows or, before
//                     the portion's start, from the request's saved tail), silu, unit norms, beta, decay
//   delta_tail        per request: the last taps - 1 raw inputs of the portion become the saved tail
//   delta_scan        per (request, head, 32 value columns): the recurrence over the portion's tokens,
//                     one value column's state spread over eight lanes' registers, inputs staged
//                     through shared memory a chunk of tokens ahead
//   delta_gated_norm  per (token, head): o / rms(o) * w * silu(gate)
//
// A request's state row is [heads][vdim][dim] floats (a column of S is contiguous) followed by the
// convolution tail [taps - 1][channels]; channels are q | k | v in the projection's column order.  A
// portion that starts at position 0 ignores what the row holds.  Every sum's order depends only on the
// token's place in its sequence, so results do not change with how a sequence is cut or batched.
#include "common.cuh"

#define DELTA_PARTS 8            // lanes that share one value column
#define DELTA_COLS 32            // value columns of a block (16 when that fills the GPU better)

// One block per (token, unit): a unit is one query head, one key head (dim channels each) or one value
// head (vdim channels, and the head's beta and decay), so that even a single token spreads over many SMs.
template <typename T, typename TW>
__global__ void __launch_bounds__(128) delta_prep_kernel(
    const T* __restrict__ proj, long ld, const TW* __restrict__ conv_w, const TW* __restrict__ a_log,
    const TW* __restrict__ dt_bias, const float* __restrict__ state, long state_stride, long tail_off,
    const int* __restrict__ tok_req, const int* __restrict__ positions, const int* __restrict__ req_ctx,
    const int* __restrict__ req_slot, float* __restrict__ work, long work_ld,
    int heads, int kv_heads, int dim, int vdim, int taps, float unit_eps, float q_scale) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float conv_out[];                      // [max(dim, vdim)]
    __shared__ float scratch[32];
    const int t = blockIdx.x, unit = blockIdx.y, tid = threadIdx.x;
    const int qk_cols = kv_heads * dim, hv = heads * vdim;
    const int channels = 2 * qk_cols + hv;
    const bool is_v = unit >= 2 * kv_heads;
    const int first = is_v ? 2 * qk_cols + (unit - 2 * kv_heads) * vdim : unit * dim;
    const int count = is_v ? vdim : dim;
    const int r = tok_req[t], pos = positions[t], ctx = req_ctx[r];
    const float* tail = state + (long)req_slot[r] * state_stride + tail_off;
    const T* row = proj + (long)t * ld;
    float ss = 0.0f;
    for (int i = tid; i < count; i += blockDim.x) {
        const int c = first + i;
        float acc = 0.0f;
        for (int back = taps - 1; back >= 0; --back) {        // oldest input first
            const int p = pos - back;
            if (p < 0) continue;
            const float x = p >= ctx ? to_f32<T>(row[c - (long)back * ld])
                                     : tail[(long)(p - ctx + taps - 1) * channels + c];
            acc += to_f32<TW>(conv_w[(long)c * taps + (taps - 1 - back)]) * x;
        }
        const float y = acc / (1.0f + expf(-acc));
        conv_out[i] = y;
        ss += y * y;
    }
    float* out_row = work + (long)t * work_ld;               // work row: q | k | v | beta | decay | o
    if (!is_v) {
        ss = block_sum(ss, scratch);
        const float f = (unit < kv_heads ? q_scale : 1.0f) / sqrtf(ss + unit_eps);
        for (int i = tid; i < count; i += blockDim.x) out_row[first + i] = conv_out[i] * f;   // each thread its own
        return;
    }
    for (int i = tid; i < count; i += blockDim.x) out_row[first + i] = conv_out[i];
    if (tid == 0) {
        const int h = unit - 2 * kv_heads;
        // two numbers a head and token, and the decay is multiplied up over thousands of tokens: formed in
        // double and rounded once, so that no bias of a float exponential adds up along a sequence
        const double b = (double)to_f32<T>(row[channels + hv + h]);
        const double a = (double)to_f32<T>(row[channels + hv + heads + h]) + (double)to_f32<TW>(dt_bias[h]);
        const double softplus = a > 30.0 ? a : log1p(exp(a));
        out_row[channels + h] = (float)(1.0 / (1.0 + exp(-b)));
        out_row[channels + heads + h] = (float)exp(-exp((double)to_f32<TW>(a_log[h])) * softplus);
    }
}

template <typename T>
__global__ void delta_tail_kernel(const T* __restrict__ proj, long ld, float* __restrict__ state, long state_stride,
                                  long tail_off, const int* __restrict__ req_start, const int* __restrict__ req_ctx,
                                  const int* __restrict__ req_qlen, const int* __restrict__ req_slot, int channels,
                                  int taps) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int start = req_start[r], ctx = req_ctx[r], qlen = req_qlen[r];
    float* tail = state + (long)req_slot[r] * state_stride + tail_off;
    // entry j holds the input at position end - (taps - 1) + j; an older entry moves down from j + qlen,
    // which lies above j, so going upwards in place is safe
    for (int j = 0; j < taps - 1; ++j) {
        const int p = ctx + qlen - (taps - 1) + j;
        float x = 0.0f;
        if (p >= ctx) x = to_f32<T>(proj[(long)(start + p - ctx) * ld + c]);
        else if (p >= 0) x = tail[(long)(j + qlen) * channels + c];
        tail[(long)j * channels + c] = x;
    }
}

// One block: one request, one head, DELTA_COLS value columns.  Thread (col, part) keeps the DPT elements
// d = part * DPT + i of column `col` of S.  The tokens' inputs (k, q of the head, the block's v columns,
// beta, decay) come through shared memory in chunks of DELTA_CHUNK tokens, the next chunk in flight
// (cp.async) while this one is consumed: the recurrence never waits for global memory.  In shared memory
// a part's k (and q) elements are contiguous and parts are DPT + 4 floats apart, so a thread fetches them
// four at a time without bank conflicts.
#define DELTA_CHUNK 16

__device__ __forceinline__ void delta_cp16(float* smem, const float* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}

__device__ __forceinline__ void delta_cp4(float* smem, const float* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem));
}

template <int DPT, int COLS, bool VEC>
__global__ void __launch_bounds__(COLS * DELTA_PARTS) delta_scan_kernel(
    float* __restrict__ work, long work_ld, float* __restrict__ state, long state_stride,
    const int* __restrict__ req_start, const int* __restrict__ req_ctx, const int* __restrict__ req_qlen,
    const int* __restrict__ req_slot, int heads, int kv_heads, int dim, int vdim) {
    static_assert(DPT % 4 == 0, "a thread's elements are fetched four at a time");
    pdl_wait();
    pdl_trigger();
    constexpr int PART = DPT + 4;                            // floats between parts
    constexpr int KQ = DELTA_PARTS * PART;                   // k (and q) of one token
    constexpr int PER_TOKEN = 2 * KQ + COLS + 4;       // k | q | v COLS | beta | decay | pad
    extern __shared__ __align__(16) float delta_in[];        // [2][DELTA_CHUNK][PER_TOKEN]
    const int r = blockIdx.x / heads, h = blockIdx.x % heads;
    const int g = h / (heads / kv_heads);
    const int part = threadIdx.x & (DELTA_PARTS - 1), col = threadIdx.x / DELTA_PARTS;
    const int j = blockIdx.y * COLS + col;
    const bool live = j < vdim;
    const int jj = live ? j : vdim - 1;                      // idle columns shadow the last one and store nothing
    const int start = req_start[r], qlen = req_qlen[r];
    float* s_col = state + (long)req_slot[r] * state_stride + ((long)h * vdim + jj) * dim;
    const int qk_cols = kv_heads * dim, hv = heads * vdim;
    const int v0 = blockIdx.y * COLS;
    if (dim < DELTA_PARTS * DPT) {                           // the k and q places beyond dim are read: they stay 0
        const int used = (qlen < DELTA_CHUNK ? qlen : 2 * DELTA_CHUNK) * PER_TOKEN;
        for (int idx = threadIdx.x; idx < used; idx += blockDim.x) delta_in[idx] = 0.0f;
        __syncthreads();
    }
    // rows whose pieces are all 16-byte aligned are copied four floats at a time, 128 slots a token
    const bool wide = dim % 4 == 0 && vdim % 4 == 0 && v0 + COLS <= vdim && dim / 2 + COLS / 4 + 2 <= 128 && work_ld % 4 == 0;
    auto fetch = [&](int buf, int first) {                   // tokens first .. first + DELTA_CHUNK - 1 of the portion
        float* dst = delta_in + (long)buf * DELTA_CHUNK * PER_TOKEN;
        const int n_tok = min(DELTA_CHUNK, qlen - first);
        if (wide) {
            const int c = threadIdx.x & 127, quarter = dim / 4;
            for (int n = threadIdx.x >> 7; n < n_tok; n += (COLS * DELTA_PARTS) >> 7) {
                const float* row = work + (long)(start + first + n) * work_ld;
                float* to = dst + (long)n * PER_TOKEN;
                if (c < 2 * quarter) {                                            // k, then q
                    const int d = (c < quarter ? c : c - quarter) * 4;
                    delta_cp16(to + (c < quarter ? 0 : KQ) + (d / DPT) * PART + d % DPT,
                               row + (c < quarter ? qk_cols : 0) + g * dim + d);
                } else if (c < 2 * quarter + COLS / 4) {
                    const int e = (c - 2 * quarter) * 4;
                    delta_cp16(to + 2 * KQ + e, row + 2 * qk_cols + h * vdim + v0 + e);
                } else if (c < 2 * quarter + COLS / 4 + 2) {                      // beta, decay
                    const int e = c - 2 * quarter - COLS / 4;
                    delta_cp4(to + 2 * KQ + COLS + e, row + 2 * qk_cols + hv + e * heads + h);
                }
            }
            asm volatile("cp.async.commit_group;");
            return;
        }
        const int wanted = 2 * dim + COLS + 2;
        for (int idx = threadIdx.x; idx < n_tok * wanted; idx += blockDim.x) {
            const int n = idx / wanted, e = idx % wanted;
            const float* row = work + (long)(start + first + n) * work_ld;
            const float* src;
            int at;
            if (e < 2 * dim) {                                                    // k, then q
                const int d = e < dim ? e : e - dim;
                src = row + (e < dim ? qk_cols : 0) + g * dim + d;
                at = (e < dim ? 0 : KQ) + (d / DPT) * PART + d % DPT;
            } else if (e < 2 * dim + COLS) {
                src = row + 2 * qk_cols + h * vdim + min(v0 + e - 2 * dim, vdim - 1);
                at = 2 * KQ + (e - 2 * dim);
            } else {                                                              // beta, decay
                src = row + 2 * qk_cols + hv + (e - 2 * dim - COLS) * heads + h;
                at = 2 * KQ + COLS + (e - 2 * dim - COLS);
            }
            delta_cp4(dst + (long)n * PER_TOKEN + at, src);
        }
        asm volatile("cp.async.commit_group;");
    };
    float S[DPT];
    const bool fresh = req_ctx[r] == 0;
    fetch(0, 0);
    // VEC (steps of single tokens, where reading and writing the state is all the work): every thread's elements
    // exist and every column starts on 16 bytes, so the state moves four floats at a time
    const bool whole = VEC && dim == DELTA_PARTS * DPT && state_stride % 4 == 0;
    if (whole && !fresh) {
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
            const float4 v = *reinterpret_cast<const float4*>(s_col + part * DPT + i);
            S[i] = v.x; S[i + 1] = v.y; S[i + 2] = v.z; S[i + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = part * DPT + i;
            S[i] = (!fresh && d < dim) ? s_col[d] : 0.0f;
        }
    }
    float* o_base = work + (long)start * work_ld + 2 * qk_cols + hv + 2 * heads + h * vdim + j;
    for (int first = 0, buf = 0; first < qlen; first += DELTA_CHUNK, buf ^= 1) {
        if (first + DELTA_CHUNK < qlen) {
            fetch(buf ^ 1, first + DELTA_CHUNK);
            asm volatile("cp.async.wait_group 1;");
        } else {
            asm volatile("cp.async.wait_group 0;");
        }
        __syncthreads();
        const float* in = delta_in + (long)buf * DELTA_CHUNK * PER_TOKEN;
        const int n_tok = min(DELTA_CHUNK, qlen - first);
        for (int n = 0; n < n_tok; ++n, in += PER_TOKEN) {
            // With a = S^T k, b = S^T q (S before the token) and c = q . k:  u = beta (v - g a) and the
            // read-out of the updated state is g b + c u.  The three sums are independent, so their chains
            // and their reductions over the column's lanes overlap; only u stands between this token's
            // sums and the next token's.
            float k[DPT], a[2] = {0.0f, 0.0f}, bq[2] = {0.0f, 0.0f}, c[2] = {0.0f, 0.0f};
#pragma unroll
            for (int i = 0; i < DPT; i += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(in + part * PART + i);
                const float4 qv = *reinterpret_cast<const float4*>(in + KQ + part * PART + i);
                k[i] = kv.x; k[i + 1] = kv.y; k[i + 2] = kv.z; k[i + 3] = kv.w;
                a[0] += S[i] * kv.x;      bq[0] += S[i] * qv.x;      c[0] += qv.x * kv.x;
                a[1] += S[i + 1] * kv.y;  bq[1] += S[i + 1] * qv.y;  c[1] += qv.y * kv.y;
                a[0] += S[i + 2] * kv.z;  bq[0] += S[i + 2] * qv.z;  c[0] += qv.z * kv.z;
                a[1] += S[i + 3] * kv.w;  bq[1] += S[i + 3] * qv.w;  c[1] += qv.w * kv.w;
            }
            float dot = a[0] + a[1], read = bq[0] + bq[1], qk = c[0] + c[1];
#pragma unroll
            for (int o = 1; o < DELTA_PARTS; o <<= 1) {
                dot += __shfl_xor_sync(0xffffffffu, dot, o);
                read += __shfl_xor_sync(0xffffffffu, read, o);
                qk += __shfl_xor_sync(0xffffffffu, qk, o);
            }
            const float decay = in[2 * KQ + COLS + 1];
            const float u = in[2 * KQ + COLS] * (in[2 * KQ + col] - decay * dot);
#pragma unroll
            for (int i = 0; i < DPT; ++i) S[i] = fmaf(k[i], u, decay * S[i]);
            if (live && part == 0) o_base[(long)(first + n) * work_ld] = decay * read + qk * u;
        }
        __syncthreads();                                     // the chunk is overwritten by the fetch after next
    }
    if (live && whole) {
#pragma unroll
        for (int i = 0; i < DPT; i += 4)
            *reinterpret_cast<float4*>(s_col + part * DPT + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
    } else if (live) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = part * DPT + i;
            if (d < dim) s_col[d] = S[i];
        }
    }
}

// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * silu(gate[t, h, :]); one warp per (token, head).
template <typename T, typename TW>
__global__ void __launch_bounds__(128) delta_gated_norm_kernel(const float* __restrict__ o, long o_ld, const T* __restrict__ gate,
                                                               long gate_ld, const TW* __restrict__ w, T* __restrict__ out,
                                                               long out_ld, int heads, int vdim, float eps) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int h = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (h >= heads) return;
    const float* x = o + (long)t * o_ld + h * vdim;
    const T* gr = gate + (long)t * gate_ld + h * vdim;
    T* dst = out + (long)t * out_ld + h * vdim;
    float ss = 0.0f;
    for (int i = lane; i < vdim; i += 32) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int i = lane; i < vdim; i += 32) {
        const float z = to_f32<T>(gr[i]);
        dst[i] = from_f32<T>(x[i] * inv * to_f32<TW>(w[i]) * (z / (1.0f + expf(-z))));
    }
}

// proj: [n_tokens, ld] with columns q | k | v | gate | b | a.
FL_API int fl_delta_prep(const void* proj, int dtype, long ld, const void* conv_w, const void* a_log, const void* dt_bias,
                         int w_dtype, float* state, long state_stride, long tail_off, const int* tok_req,
                         const int* positions, const int* req_start, const int* req_ctx, const int* req_qlen,
                         const int* req_slot, float* work, long work_ld, int n_tokens, int n_requests,
                         int heads, int kv_heads, int dim, int vdim, int taps, float unit_eps, float q_scale,
                         cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int channels = 2 * kv_heads * dim + heads * vdim;
    const int units = 2 * kv_heads + heads, widest = dim > vdim ? dim : vdim;
    if (taps < 1 || heads % kv_heads || n_requests > 65535 || units > 65535 || (size_t)widest * sizeof(float) > 48 * 1024)
        return (int)cudaErrorInvalidValue;
    int rc = 0;
    FL_DISPATCH(dtype, T, FL_DISPATCH(w_dtype, TW,
        rc = fl_launch(delta_prep_kernel<T, TW>, dim3(n_tokens, units), dim3(128), (size_t)widest * sizeof(float), stream,
                       (const T*)proj, ld, (const TW*)conv_w, (const TW*)a_log, (const TW*)dt_bias, (const float*)state,
                       state_stride, tail_off, tok_req, positions, req_ctx, req_slot, work, work_ld, heads, kv_heads,
                       dim, vdim, taps, unit_eps, q_scale)));
    if (rc || taps == 1) return rc;
    FL_DISPATCH(dtype, T,
        return fl_launch(delta_tail_kernel<T>, dim3((channels + 255) / 256, n_requests), dim3(256), 0, stream,
                         (const T*)proj, ld, state, state_stride, tail_off, req_start, req_ctx, req_qlen, req_slot,
                         channels, taps));
    return 0;
}

// single_tokens: every request of the step brings one token (the state then moves in 16-byte pieces).
// work: [n_tokens, work_ld] floats, a row = q | k (kv_heads x dim each) | v (heads x vdim) | beta | decay (heads
// each) | o (heads x vdim): fl_delta_prep fills all but o, fl_delta_scan reads them and fills o.
FL_API int fl_delta_scan(float* work, long work_ld, float* state, long state_stride,
                         const int* req_start, const int* req_ctx, const int* req_qlen, const int* req_slot,
                         int n_requests, int heads, int kv_heads, int dim, int vdim, int single_tokens, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (heads % kv_heads || dim < 1 || dim > 32 * DELTA_PARTS) return (int)cudaErrorInvalidValue;
    const int per_thread = (dim + DELTA_PARTS - 1) / DELTA_PARTS;
    // a block takes 32 value columns, or 16 when blocks of 32 would leave most of the GPU idle (a lone
    // request's prompt): the recurrence is a chain per token, so what counts is how many SMs walk it
    const bool narrow = (long)n_requests * heads * ((vdim + 31) / 32) < 96 && vdim > 16;
    const int cols = narrow ? 16 : DELTA_COLS;
    dim3 grid(n_requests * heads, (vdim + cols - 1) / cols);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
#define FL_DELTA_SCAN_COLS(DPT, COLS, VEC)                                                                          \
    {                                                                                                               \
        const size_t smem = (size_t)2 * DELTA_CHUNK * (2 * DELTA_PARTS * (DPT + 4) + COLS + 4) * sizeof(float);     \
        static bool raised = false;                                                                                 \
        if (smem > 48 * 1024 && !raised) {                                                                          \
            const cudaError_t rc = cudaFuncSetAttribute(delta_scan_kernel<DPT, COLS, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (rc != cudaSuccess) return (int)rc;                                                                  \
            raised = true;                                                                                          \
        }                                                                                                           \
        return fl_launch(delta_scan_kernel<DPT, COLS, VEC>, grid, dim3(COLS * DELTA_PARTS), smem, stream, work, work_ld, state, \
                         state_stride, req_start, req_ctx, req_qlen, req_slot, heads, kv_heads, dim, vdim);         \
    }
#define FL_DELTA_SCAN(DPT)                                                                                          \
    if (per_thread <= DPT) {                                                                                        \
        if (single_tokens) { if (narrow) FL_DELTA_SCAN_COLS(DPT, 16, true) else FL_DELTA_SCAN_COLS(DPT, 32, true) }  \
        else { if (narrow) FL_DELTA_SCAN_COLS(DPT, 16, false) else FL_DELTA_SCAN_COLS(DPT, 32, false) }             \
    }
    FL_DELTA_SCAN(4);
    FL_DELTA_SCAN(8);
    FL_DELTA_SCAN(12);
    FL_DELTA_SCAN(16);
    FL_DELTA_SCAN(24);
    FL_DELTA_SCAN(32);
#undef FL_DELTA_SCAN_COLS
#undef FL_DELTA_SCAN
    return (int)cudaErrorInvalidValue;
}

FL_API int fl_delta_gated_norm(const float* o, long o_ld, const void* gate, int dtype, long gate_ld, const void* w, int w_dtype,
                               void* out, long out_ld, int n_tokens, int heads, int vdim, float eps, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    dim3 grid(n_tokens, (heads + 3) / 4);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(dtype, T, FL_DISPATCH(w_dtype, TW,
        return fl_launch(delta_gated_norm_kernel<T, TW>, grid, dim3(128), 0, stream, o, o_ld, (const T*)gate, gate_ld,
                         (const TW*)w, (T*)out, out_ld, heads, vdim, eps)));
    return 0;
}
