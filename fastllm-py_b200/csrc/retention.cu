// Retention: linear attention with a fixed decay per head and no softmax or denominator.
//
// Per head, with a state S [dim x vdim] in float that a request carries from token to token:
//     S <- decay S + k v^T;   o = S^T q
// q and k are rotated (pairs (i, i + rot/2) of the first `rot` dimensions) and k is multiplied by
// `k_scale` after the rotation.  The head's o is divided by its root mean square and multiplied by
// silu(gate).
//
//   retention_prep        per (token, q or k head): rotation and scale into a float work row q | k
//   retention_scan        per (request, head, 32 value columns): the recurrence over the portion's tokens,
//                         one value column's state spread over eight lanes' registers, the tokens' q, k and
//                         v staged through shared memory a chunk at a time
//   retention_gated_norm  per (token, head): o / sqrt(mean(o^2) + eps) * silu(gate)
//
// A request's state row is [heads][vdim][dim] floats (a column of S is contiguous).  A portion that
// starts at position 0 ignores what the row holds.  The read-out sums a column's dim products in a
// fixed order, so results do not change with how a sequence is cut or batched.  Everything after the
// projections is float.
#include "common.cuh"

#define RET_PARTS 8              // lanes that share one value column
#define RET_COLS 32              // value columns of a block
#define RET_CHUNK 16             // tokens staged at a time

template <typename T>
__global__ void __launch_bounds__(128) retention_prep_kernel(
    const T* __restrict__ proj, long ld, float* __restrict__ work, long work_ld, int heads, int dim, int rot,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, const int* __restrict__ positions,
    float k_scale) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, unit = blockIdx.y;           // units: q heads, then k heads, in the projection's order
    const int half = rot >> 1;
    const long pos = positions[t];
    const float* cs = cos_table + pos * half;
    const float* sn = sin_table + pos * half;
    const T* x = proj + (long)t * ld + (long)unit * dim;
    float* y = work + (long)t * work_ld + (long)unit * dim;
    const float f = unit < heads ? 1.0f : k_scale;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float a = to_f32<T>(x[j]), b = to_f32<T>(x[j + half]);
        y[j] = (a * cs[j] - b * sn[j]) * f;
        y[j + half] = (b * cs[j] + a * sn[j]) * f;
    }
    for (int j = rot + threadIdx.x; j < dim; j += blockDim.x) y[j] = to_f32<T>(x[j]) * f;
}

// proj columns: q (heads x dim) | k (heads x dim) | ...; work columns: q | k (float).
FL_API int fl_retention_prep(const void* proj, int dtype, long ld, float* work, long work_ld, int n_tokens, int heads,
                             int dim, int rot, const float* cos_table, const float* sin_table, const int* positions,
                             float k_scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot < 0 || rot > dim || (rot & 1) || 2 * heads > 65535) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(dtype, T, return fl_launch(retention_prep_kernel<T>, dim3(n_tokens, 2 * heads), dim3(128), 0, stream,
                                           (const T*)proj, ld, work, work_ld, heads, dim, rot, cos_table, sin_table,
                                           positions, k_scale));
    return 0;
}

// NI: state elements per lane (dim <= 8 NI).  A lane holds rows part, part + 8, ... of its column.
template <typename T, int NI>
__global__ void __launch_bounds__(RET_COLS * RET_PARTS) retention_scan_kernel(
    const float* __restrict__ qk, long qk_ld, const T* __restrict__ v, long v_ld, float* __restrict__ o, long o_ld,
    float* __restrict__ state, long state_stride, const float* __restrict__ decay, const int* __restrict__ req_start,
    const int* __restrict__ req_ctx, const int* __restrict__ req_qlen, const int* __restrict__ req_slot, int heads,
    int dim, int vdim) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float ret_smem[];                    // [CHUNK][2 dim] q | k, then [CHUNK][COLS] v
    float* qk_s = ret_smem;
    float* v_s = ret_smem + RET_CHUNK * 2 * dim;
    const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * RET_COLS;
    const int tid = threadIdx.x, part = tid & (RET_PARTS - 1), col = col0 + (tid >> 3);
    const int start = req_start[r], qlen = req_qlen[r];
    const bool live = col < vdim;
    float* srow = state + (long)req_slot[r] * state_stride + ((long)h * vdim + (live ? col : 0)) * dim;
    float S[NI];
    const bool fresh = req_ctx[r] == 0;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int d = part + i * RET_PARTS;
        S[i] = (!fresh && live && d < dim) ? srow[d] : 0.0f;
    }
    const float g = decay[h];
    for (int base = 0; base < qlen; base += RET_CHUNK) {
        const int n = min(RET_CHUNK, qlen - base);
        __syncthreads();                                   // the chunk before is read out
        for (int i = tid; i < n * 2 * dim; i += blockDim.x) {
            const int c = i / (2 * dim), e = i - c * 2 * dim;
            const int which = e / dim, d = e - which * dim;
            qk_s[i] = qk[(long)(start + base + c) * qk_ld + (long)which * heads * dim + (long)h * dim + d];
        }
        for (int i = tid; i < n * RET_COLS; i += blockDim.x) {
            const int c = i / RET_COLS, j = i - c * RET_COLS;
            v_s[i] = col0 + j < vdim ? to_f32<T>(v[(long)(start + base + c) * v_ld + (long)h * vdim + col0 + j]) : 0.0f;
        }
        __syncthreads();
        for (int c = 0; c < n; ++c) {
            const float* qs = qk_s + c * 2 * dim;
            const float* ks = qs + dim;
            const float vj = v_s[c * RET_COLS + (tid >> 3)];
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int d = part + i * RET_PARTS;
                if (d < dim) {
                    S[i] = g * S[i] + ks[d] * vj;
                    acc += S[i] * qs[d];
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (part == 0 && live) o[(long)(start + base + c) * o_ld + (long)h * vdim + col] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int d = part + i * RET_PARTS;
            if (d < dim) srow[d] = S[i];
        }
    }
}

// qk: float [n_tokens, qk_ld] with columns q (heads x dim) | k (heads x dim), rotated and scaled; v: the value columns
// of the projection ([n_tokens, v_ld], head h at h * vdim); o: float [n_tokens, o_ld]; state: [slots, state_stride].
FL_API int fl_retention_scan(const float* qk, long qk_ld, const void* v, int v_dtype, long v_ld, float* o, long o_ld,
                             float* state, long state_stride, const float* decay, const int* req_start,
                             const int* req_ctx, const int* req_qlen, const int* req_slot, int n_requests, int heads,
                             int dim, int vdim, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    const int col_blocks = (vdim + RET_COLS - 1) / RET_COLS;
    if (dim < 1 || dim > 256 || heads > 65535 || col_blocks > 65535) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)RET_CHUNK * (2 * dim + RET_COLS) * sizeof(float);
    dim3 grid(n_requests, heads, col_blocks), block(RET_COLS * RET_PARTS);
#define FL_RET_SCAN(NI)                                                                                              \
    FL_DISPATCH(v_dtype, T, return fl_launch(retention_scan_kernel<T, NI>, grid, block, smem, stream, qk, qk_ld,     \
                                             (const T*)v, v_ld, o, o_ld, state, state_stride, decay, req_start,      \
                                             req_ctx, req_qlen, req_slot, heads, dim, vdim))
    if (dim <= 32) { FL_RET_SCAN(4); }
    else if (dim <= 64) { FL_RET_SCAN(8); }
    else if (dim <= 128) { FL_RET_SCAN(16); }
    else { FL_RET_SCAN(32); }
#undef FL_RET_SCAN
    return 0;
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * silu(gate[t, h, :]); one warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128) retention_gated_norm_kernel(const float* __restrict__ o, long o_ld,
                                                                   const T* __restrict__ gate, long gate_ld,
                                                                   T* __restrict__ out, long out_ld, int heads, int vdim,
                                                                   float eps) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int h = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (h >= heads) return;
    const float* x = o + (long)t * o_ld + (long)h * vdim;
    const T* gr = gate + (long)t * gate_ld + (long)h * vdim;
    T* dst = out + (long)t * out_ld + (long)h * vdim;
    float ss = 0.0f;
    for (int i = lane; i < vdim; i += 32) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int i = lane; i < vdim; i += 32) {
        const float z = to_f32<T>(gr[i]);
        dst[i] = from_f32<T>(x[i] * inv * (z / (1.0f + expf(-z))));
    }
}

FL_API int fl_retention_gated_norm(const float* o, long o_ld, const void* gate, int dtype, long gate_ld, void* out,
                                   long out_ld, int n_tokens, int heads, int vdim, float eps, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    dim3 grid(n_tokens, (heads + 3) / 4);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(dtype, T, return fl_launch(retention_gated_norm_kernel<T>, grid, dim3(128), 0, stream, o, o_ld,
                                           (const T*)gate, gate_ld, (T*)out, out_ld, heads, vdim, eps));
    return 0;
}
