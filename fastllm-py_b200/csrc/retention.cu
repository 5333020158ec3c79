// Retention: linear attention with a fixed decay per head and no softmax or denominator.
//
// Per head, with a state S [dim x vdim] in float that a request carries from token to token:
//     S <- decay S + k v^T;   o = S^T q
// q and k are rotated (pairs (i, i + rot/2) of the first `rot` dimensions) and k is multiplied by
// `k_scale` after the rotation.  The head's o is divided by its root mean square and multiplied by
// silu(gate).
//
//   retention_prep        per token: rotation and scale of every head into a float work row q | k | v
//   retention_scan        per (request, head, 32, 16 or 8 value columns): the recurrence over the portion's tokens,
//                         one value column's state spread over the registers of 8, 16 or 32 lanes, the tokens'
//                         q, k and v staged through shared memory a chunk of 16 ahead (cp.async, two buffers),
//                         four tokens side by side
//   retention_gated_norm  per (token, head): o / sqrt(mean(o^2) + eps) * silu(gate)
//
// A request's state row is [heads][vdim][dim] floats (a column of S is contiguous).  A portion that
// starts at position 0 ignores what the row holds.  For a given number of lanes a column the read-out
// sums a column's dim products in a fixed order with fixed roundings, so results do not change with
// how a sequence is cut or batched; the launcher's `fixed_order` keeps that number at eight whatever
// the step's shape (the 32-bit path), otherwise a lone prompt takes more lanes than a batch and the
// two differ by rounding.  Everything after the projections is float.
#include "common.cuh"

#define RET_CHUNK 16             // tokens staged at a time

// One block per token: the rotated pairs of every q and k head, what lies behind them, and the values.
template <typename T>
__global__ void __launch_bounds__(256) retention_prep_kernel(
    const T* __restrict__ proj, long ld, float* __restrict__ work, long work_ld, int heads, int dim, int vdim, int rot,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, const int* __restrict__ positions,
    float k_scale) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = rot >> 1;
    const long pos = positions[t];
    const float* cs = cos_table + pos * half;
    const float* sn = sin_table + pos * half;
    const T* x = proj + (long)t * ld;
    float* y = work + (long)t * work_ld;
    for (int i = threadIdx.x; i < 2 * heads * half; i += blockDim.x) {
        const int unit = i / half, j = i - unit * half;     // units: q heads, then k heads, in the projection's order
        const float f = unit < heads ? 1.0f : k_scale;
        const long at = (long)unit * dim + j;
        const float a = to_f32<T>(x[at]), b = to_f32<T>(x[at + half]);
        y[at] = (a * cs[j] - b * sn[j]) * f;
        y[at + half] = (b * cs[j] + a * sn[j]) * f;
    }
    const int rest = dim - rot;
    for (int i = threadIdx.x; i < 2 * heads * rest; i += blockDim.x) {
        const int unit = i / rest;
        const long at = (long)unit * dim + rot + (i - unit * rest);
        y[at] = to_f32<T>(x[at]) * (unit < heads ? 1.0f : k_scale);
    }
    const long v0 = (long)2 * heads * dim;
    for (int i = threadIdx.x; i < heads * vdim; i += blockDim.x) y[v0 + i] = to_f32<T>(x[v0 + i]);   // widened as they are
}

// proj columns: q (heads x dim) | k (heads x dim) | v (heads x vdim) | ...; work columns: q | k | v (float).
FL_API int fl_retention_prep(const void* proj, int dtype, long ld, float* work, long work_ld, int n_tokens, int heads,
                             int dim, int vdim, int rot, const float* cos_table, const float* sin_table,
                             const int* positions, float k_scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot < 0 || rot > dim || (rot & 1)) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(dtype, T, return fl_launch(retention_prep_kernel<T>, dim3(n_tokens), dim3(256), 0, stream,
                                           (const T*)proj, ld, work, work_ld, heads, dim, vdim, rot, cos_table,
                                           sin_table, positions, k_scale));
    return 0;
}

__device__ __forceinline__ void ret_cp(float* dst, const float* src, int bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

// One state element's step: S <- g S + k v, then the read-out's sum takes S q.  Written with explicit roundings so
// that every path through the kernel (four tokens at a time, a portion's last tokens one by one) does the same
// arithmetic: a token's result does not depend on where a portion was cut.
__device__ __forceinline__ void ret_update(float& S, float& acc, float g, float k, float q, float v) {
    S = __fmaf_rn(g, S, __fmul_rn(k, v));
    acc = __fmaf_rn(S, q, acc);
}

// PARTS: lanes that share one value column (8, 16 or 32); NI: state elements per lane (dim <= PARTS * NI, a multiple
// of 4); COLS: value columns of a block.  A staged token is dim floats of q, dim of k and COLS of v; with VEC
// every staged piece starts 16 bytes aligned (dim and vdim multiples of 4) and rows are read four floats at a time;
// FULL: dim == PARTS * NI, so no lane's rows lie beyond dim and the loads have no bounds to test.
// Lane `part` holds, of its column, rows (i / 4) * 4 PARTS + part * 4 + i % 4: four neighbours at a time, so that
// the lanes of a column read consecutive bytes of a staged q or k row with one 16-byte load each.
template <int NI, int COLS, int PARTS, bool VEC, bool FULL>
__global__ void __launch_bounds__(COLS * PARTS) retention_scan_kernel(
    const float* __restrict__ qkv, long ld, float* __restrict__ o, long o_ld, float* __restrict__ state,
    long state_stride, const float* __restrict__ decay, const int* __restrict__ req_start,
    const int* __restrict__ req_ctx, const int* __restrict__ req_qlen, const int* __restrict__ req_slot, int heads,
    int dim, int vdim) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) float ret_smem[];      // two buffers of [CHUNK][2 dim + COLS]
    const int row_w = 2 * dim + COLS;
    const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
    const int tid = threadIdx.x, part = tid % PARTS, col = col0 + tid / PARTS;
    const int start = req_start[r], qlen = req_qlen[r];
    const bool live = col < vdim;
    float* srow = state + (long)req_slot[r] * state_stride + ((long)h * vdim + (live ? col : 0)) * dim;
    float S[NI];
    const bool fresh = req_ctx[r] == 0;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int d = (i >> 2) * (4 * PARTS) + part * 4 + (i & 3);
        S[i] = (!fresh && live && d < dim) ? srow[d] : 0.0f;
    }
    const float g = decay[h];
    const long q_off = (long)h * dim, k_off = (long)heads * dim + (long)h * dim;
    const long v_off = (long)2 * heads * dim + (long)h * vdim + col0;
    const int v_cols = min(COLS, vdim - col0);

    // stage chunk `base` into buffer `buf`
    auto stage = [&](int base, int buf) {
        float* dst = ret_smem + (long)buf * RET_CHUNK * row_w;
        const int n = min(RET_CHUNK, qlen - base);
        if (VEC) {
            const int per = row_w / 4, qk4 = dim / 4;
            for (int i = tid; i < n * per; i += blockDim.x) {
                const int c = i / per, e = i - c * per;
                const float* src = qkv + (long)(start + base + c) * ld;
                if (e < qk4) src += q_off + e * 4;
                else if (e < 2 * qk4) src += k_off + (e - qk4) * 4;
                else if ((e - 2 * qk4) * 4 < v_cols) src += v_off + (e - 2 * qk4) * 4;
                else continue;
                ret_cp(dst + c * row_w + e * 4, src, 16);
            }
        } else {
            for (int i = tid; i < n * row_w; i += blockDim.x) {
                const int c = i / row_w, e = i - c * row_w;
                const float* src = qkv + (long)(start + base + c) * ld;
                if (e < dim) src += q_off + e;
                else if (e < 2 * dim) src += k_off + (e - dim);
                else if (e - 2 * dim < v_cols) src += v_off + (e - 2 * dim);
                else continue;
                ret_cp(dst + c * row_w + e, src, 4);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // the four (or fewer) state rows of group i4 that token row `rowp` (q at 0, k at dim) holds for this lane
    auto fetch = [&](const float* rowp, int i4, float* out4) {
        const int d0 = i4 * (4 * PARTS) + part * 4;
        if (VEC && FULL) {
            const float4 v = reinterpret_cast<const float4*>(rowp)[i4 * PARTS + part];
            out4[0] = v.x; out4[1] = v.y; out4[2] = v.z; out4[3] = v.w;
        } else if (VEC) {
            const float4 v = d0 < dim ? *reinterpret_cast<const float4*>(rowp + d0) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            out4[0] = v.x; out4[1] = v.y; out4[2] = v.z; out4[3] = v.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) out4[e] = d0 + e < dim ? rowp[d0 + e] : 0.0f;     // (rows beyond dim add nothing)
        }
    };

    stage(0, 0);
    int buf = 0;
    for (int base = 0; base < qlen; base += RET_CHUNK, buf ^= 1) {
        const int n = min(RET_CHUNK, qlen - base);
        if (base + RET_CHUNK < qlen) {
            stage(base + RET_CHUNK, buf ^ 1);              // (its buffer was read out before the last barrier)
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* rows = ret_smem + (long)buf * RET_CHUNK * row_w;
        const float* mine = rows + 2 * dim + tid / PARTS;   // this column's value of the chunk's first token
        float* o_at = o + (long)(start + base) * o_ld + (long)h * vdim + col;
        // Four tokens at a time, written out so that only the state's own chain (one multiply-add a token) stands
        // between them: the tokens' read-out sums and their reductions over the lanes run side by side.  A
        // portion's last one to three tokens go one by one, with the same arithmetic.
        for (int c0 = 0; c0 < n; c0 += 4) {
            const int m = min(4, n - c0);
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, vj[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) vj[u] = (live && u < m) ? mine[(c0 + u) * row_w] : 0.0f;
            if (m == 4) {
#pragma unroll
                for (int i4 = 0; i4 < NI / 4; ++i4) {
                    float kv[4][4], qv[4][4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float* rowp = rows + (c0 + u) * row_w;
                        fetch(rowp, i4, qv[u]);
                        fetch(rowp + dim, i4, kv[u]);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int e = 0; e < 4; ++e) ret_update(S[i4 * 4 + e], acc[u], g, kv[u][e], qv[u][e], vj[u]);
                }
            } else {
                for (int u = 0; u < m; ++u) {
                    const float* rowp = rows + (c0 + u) * row_w;
                    const float vu = live ? mine[(c0 + u) * row_w] : 0.0f;
                    float a = 0.0f;
#pragma unroll
                    for (int i4 = 0; i4 < NI / 4; ++i4) {
                        float kk[4], qq[4];
                        fetch(rowp, i4, qq);
                        fetch(rowp + dim, i4, kk);
#pragma unroll
                        for (int e = 0; e < 4; ++e) ret_update(S[i4 * 4 + e], a, g, kk[e], qq[e], vu);
                    }
                    if (u == 0) acc[0] = a;
                    else if (u == 1) acc[1] = a;
                    else acc[2] = a;
                }
            }
#pragma unroll
            for (int o_ = 1; o_ < PARTS; o_ <<= 1)
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o_);
            if (part == 0 && live) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (u < m) o_at[(long)(c0 + u) * o_ld] = acc[u];
            }
        }
        __syncthreads();                                   // the buffer is staged into again next round
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int d = (i >> 2) * (4 * PARTS) + part * 4 + (i & 3);
            if (d < dim) srow[d] = S[i];
        }
    }
}

template <int NI, int COLS, int PARTS, bool VEC, bool FULL>
static int launch_ret_scan_as(dim3 grid, size_t smem, cudaStream_t stream, const float* qkv, long ld, float* o, long o_ld,
                              float* state, long state_stride, const float* decay, const int* req_start,
                              const int* req_ctx, const int* req_qlen, const int* req_slot, int heads, int dim, int vdim) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(retention_scan_kernel<NI, COLS, PARTS, VEC, FULL>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return fl_launch(retention_scan_kernel<NI, COLS, PARTS, VEC, FULL>, grid, dim3(COLS * PARTS), smem, stream, qkv, ld, o,
                     o_ld, state, state_stride, decay, req_start, req_ctx, req_qlen, req_slot, heads, dim, vdim);
}

template <int NI, int COLS, int PARTS>
static int launch_ret_scan(dim3 grid, size_t smem, cudaStream_t stream, const float* qkv, long ld, float* o, long o_ld,
                           float* state, long state_stride, const float* decay, const int* req_start, const int* req_ctx,
                           const int* req_qlen, const int* req_slot, int heads, int dim, int vdim, int vec) {
    if (vec && dim == NI * PARTS)
        return launch_ret_scan_as<NI, COLS, PARTS, true, true>(grid, smem, stream, qkv, ld, o, o_ld, state, state_stride,
                                                               decay, req_start, req_ctx, req_qlen, req_slot, heads, dim,
                                                               vdim);
    if (vec)
        return launch_ret_scan_as<NI, COLS, PARTS, true, false>(grid, smem, stream, qkv, ld, o, o_ld, state, state_stride,
                                                                decay, req_start, req_ctx, req_qlen, req_slot, heads, dim,
                                                                vdim);
    return launch_ret_scan_as<NI, COLS, PARTS, false, false>(grid, smem, stream, qkv, ld, o, o_ld, state, state_stride, decay,
                                                      req_start, req_ctx, req_qlen, req_slot, heads, dim, vdim);
}

// qkv: float [n_tokens, ld] with columns q (heads x dim) | k (heads x dim) | v (heads x vdim), q and k rotated and
// scaled; o: float [n_tokens, o_ld]; state: [slots, state_stride].  Blocks of 32 columns with eight lanes a column;
// when those would leave SMs idle (a lone prompt), narrower blocks with more lanes a column (16 columns x 16
// lanes for keys of 64 and more; 8 columns x 32 lanes for keys of 128 and more if SMs would still idle), so that
// more warps share a token's chain.  The lanes of a column fix the order of the read-out's sum: with `fixed_order`
// there are always eight, so that a token's result never depends on what else is in the step.
FL_API int fl_retention_scan(const float* qkv, long ld, float* o, long o_ld, float* state, long state_stride,
                             const float* decay, const int* req_start, const int* req_ctx, const int* req_qlen,
                             const int* req_slot, int n_requests, int heads, int dim, int vdim, int num_sms,
                             int fixed_order, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (dim < 1 || dim > 256 || heads > 65535) return (int)cudaErrorInvalidValue;
    const long units = (long)n_requests * heads;
    int cols = 32, parts = 8;
    if (units * ((vdim + 31) / 32) < num_sms && vdim > 16) {
        cols = 16;
        if (dim >= 64 && !fixed_order) parts = 16;
        if (dim >= 128 && !fixed_order && units * ((vdim + 15) / 16) < 2 * num_sms && vdim > 8) { cols = 8; parts = 32; }
    }
    const int col_blocks = (vdim + cols - 1) / cols;
    if (col_blocks > 65535) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)2 * RET_CHUNK * (2 * dim + cols) * sizeof(float);
    const int vec = dim % 4 == 0 && vdim % 4 == 0 && ld % 4 == 0 && ((uintptr_t)qkv % 16) == 0;
    dim3 grid(n_requests, heads, col_blocks);
#define FL_RET_ARGS grid, smem, stream, qkv, ld, o, o_ld, state, state_stride, decay, req_start, req_ctx, req_qlen, \
                    req_slot, heads, dim, vdim, vec
    if (parts == 32) {
        if (dim <= 128) return launch_ret_scan<4, 8, 32>(FL_RET_ARGS);
        return launch_ret_scan<8, 8, 32>(FL_RET_ARGS);
    }
    if (parts == 16) {
        if (dim <= 64) return launch_ret_scan<4, 16, 16>(FL_RET_ARGS);
        if (dim <= 128) return launch_ret_scan<8, 16, 16>(FL_RET_ARGS);
        return launch_ret_scan<16, 16, 16>(FL_RET_ARGS);
    }
    if (cols == 16) {
        if (dim <= 32) return launch_ret_scan<4, 16, 8>(FL_RET_ARGS);
        if (dim <= 64) return launch_ret_scan<8, 16, 8>(FL_RET_ARGS);
        if (dim <= 128) return launch_ret_scan<16, 16, 8>(FL_RET_ARGS);
        return launch_ret_scan<32, 16, 8>(FL_RET_ARGS);
    }
    if (dim <= 32) return launch_ret_scan<4, 32, 8>(FL_RET_ARGS);
    if (dim <= 64) return launch_ret_scan<8, 32, 8>(FL_RET_ARGS);
    if (dim <= 128) return launch_ret_scan<16, 32, 8>(FL_RET_ARGS);
    return launch_ret_scan<32, 32, 8>(FL_RET_ARGS);
#undef FL_RET_ARGS
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
