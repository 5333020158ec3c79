// Differential attention over a paged cache: two softmax maps per head over the same values.
//
// A query head carries two maps (q1, q2 of `dim` each, side by side), a key/value head two key maps
// (k1, k2) and one value of `vdim`.  With a_m = softmax(q_m . k_m * scale) V over the visible keys
// (those at or before the query and, with a window, the last `window` of them):
//     o = a_1 - lambda a_2;   out = o / sqrt(mean(o^2) + eps) * out_scale
// lambda is one number per layer (made by the caller), out_scale is 1 - (the layer's constant).
// Rotary pairs (i, i + rot/2) turn the first `rot` dimensions of every map of q and k.
//
// A cache page is [kv_heads, page_size, 2 dim + vdim]: a token's two key maps, then its value.
//
//   diff_prep            per (token, head): rotates the query maps in place; rotates the key maps
//                        into the token's cache row and copies the value behind them
//   diff_attention_simt  per (token, query head): CUDA cores, any sizes, bfloat16 or true 32-bit;
//                        key tiles start at multiples of 128 of the absolute position, so every sum's
//                        order depends on the token's own position only (cuts and batches agree bit
//                        for bit)
//
// Scores, softmax, the difference and the norm are float.
#include "common.cuh"

#define DIFF_TILE 128

template <typename T>
__global__ void __launch_bounds__(128) diff_prep_kernel(
    T* __restrict__ proj, long ld, int heads, int kv_heads, int dim, int vdim, int rot,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, const int* __restrict__ positions,
    const int* __restrict__ slots, T* __restrict__ cache, long page_stride, int page_size) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, unit = blockIdx.y;
    const int half = rot >> 1;
    const long pos = positions[t];
    const float* cs = cos_table + pos * half;
    const float* sn = sin_table + pos * half;
    T* row = proj + (long)t * ld;
    if (unit < heads) {                                    // both maps of a query head, in place
        T* x = row + (long)unit * 2 * dim;
        for (int i = threadIdx.x; i < 2 * half; i += blockDim.x) {
            const int m = i / half, j = i - m * half;
            T* xm = x + m * dim;
            const float a = to_f32<T>(xm[j]), b = to_f32<T>(xm[j + half]);
            xm[j] = from_f32<T>(a * cs[j] - b * sn[j]);
            xm[j + half] = from_f32<T>(b * cs[j] + a * sn[j]);
        }
        return;
    }
    if (cache == nullptr) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int g = unit - heads;
    const long page = slot / page_size;
    const int off = slot - (int)page * page_size;
    const int row_w = 2 * dim + vdim;
    T* dst = cache + page * page_stride + ((long)g * page_size + off) * row_w;
    const T* k = row + (long)heads * 2 * dim + (long)g * 2 * dim;
    const T* v = row + (long)(heads + kv_heads) * 2 * dim + (long)g * vdim;
    for (int i = threadIdx.x; i < 2 * half; i += blockDim.x) {
        const int m = i / half, j = i - m * half;
        const float a = to_f32<T>(k[m * dim + j]), b = to_f32<T>(k[m * dim + j + half]);
        dst[m * dim + j] = from_f32<T>(a * cs[j] - b * sn[j]);
        dst[m * dim + j + half] = from_f32<T>(b * cs[j] + a * sn[j]);
    }
    for (int i = threadIdx.x; i < 2 * (dim - rot); i += blockDim.x) {
        const int m = i / (dim - rot), j = rot + i - m * (dim - rot);
        dst[m * dim + j] = k[m * dim + j];
    }
    for (int i = threadIdx.x; i < vdim; i += blockDim.x) dst[2 * dim + i] = v[i];
}

// proj: [n_tokens, ld] with columns q (heads x 2 x dim) | k (kv_heads x 2 x dim) | v (kv_heads x vdim);
// cache (one layer's pages) may be null: the queries only are turned then.
FL_API int fl_diff_prep(void* proj, int dtype, long ld, int n_tokens, int heads, int kv_heads, int dim, int vdim, int rot,
                        const float* cos_table, const float* sin_table, const int* positions, const int* slots,
                        void* cache, long page_stride, int page_size, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot < 0 || rot > dim || (rot & 1) || heads + kv_heads > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid(n_tokens, heads + kv_heads);
    FL_DISPATCH(dtype, T, return fl_launch(diff_prep_kernel<T>, grid, dim3(128), 0, stream, (T*)proj, ld, heads, kv_heads,
                                           dim, vdim, rot, cos_table, sin_table, positions, slots, (T*)cache,
                                           page_stride, page_size));
    return 0;
}

template <typename T>
__global__ void __launch_bounds__(DIFF_TILE) diff_attention_simt_kernel(
    const T* __restrict__ q, long q_ld, T* __restrict__ out, long out_ld, const T* __restrict__ cache, long page_stride,
    int page_size, const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tok_req,
    const int* __restrict__ positions, int heads, int kv_heads, int dim, int vdim, int window, float scale,
    float lambda, float eps, float out_scale) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) unsigned char diff_smem[];
    long* off_s = reinterpret_cast<long*>(diff_smem);                 // [TILE] element offset of each key row
    float* p1_s = reinterpret_cast<float*>(off_s + DIFF_TILE);        // [TILE] numerators of map 1
    float* p2_s = p1_s + DIFF_TILE;                                   // [TILE] numerators of map 2
    float* q_s = p2_s + DIFF_TILE;                                    // [2 dim]
    __shared__ float scratch[32];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int g = h / (heads / kv_heads);
    const int pos = positions[t];
    const int* bt = block_table + (long)tok_req[t] * bt_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int row_w = 2 * dim + vdim;

    const T* qr = q + (long)t * q_ld + (long)h * 2 * dim;
    for (int d = tid; d < 2 * dim; d += DIFF_TILE) q_s[d] = to_f32<T>(qr[d]);
    __syncthreads();

    float m1 = -CUDART_INF_F, m2 = -CUDART_INF_F, l1 = 0.0f, l2 = 0.0f;
    float a1[2] = {0.0f, 0.0f}, a2[2] = {0.0f, 0.0f};                  // value columns tid and tid + TILE
    for (int tile = (lo / DIFF_TILE) * DIFF_TILE; tile <= pos; tile += DIFF_TILE) {
        const int j = tile + tid;
        const bool valid = j >= lo && j <= pos;
        float s1 = -CUDART_INF_F, s2 = -CUDART_INF_F;
        long off = 0;
        if (valid) {
            const long page = bt[j / page_size];
            off = page * page_stride + ((long)g * page_size + j % page_size) * row_w;
            const T* kp = cache + off;
            float d1 = 0.0f, d2 = 0.0f;
            for (int d = 0; d < dim; ++d) {
                d1 += q_s[d] * to_f32<T>(kp[d]);
                d2 += q_s[dim + d] * to_f32<T>(kp[dim + d]);
            }
            s1 = d1 * scale;
            s2 = d2 * scale;
        }
        off_s[tid] = off + 2 * dim;                       // the row's value part
        const float n1 = fmaxf(m1, block_max(s1, scratch));
        const float n2 = fmaxf(m2, block_max(s2, scratch));
        const float p1 = valid ? expf(s1 - n1) : 0.0f;
        const float p2 = valid ? expf(s2 - n2) : 0.0f;
        p1_s[tid] = p1;
        p2_s[tid] = p2;
        const float sum1 = block_sum(p1, scratch);        // its barriers also publish p1_s / p2_s / off_s
        const float sum2 = block_sum(p2, scratch);
        const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);   // 0 at the first tile (m = -inf)
        l1 = l1 * c1 + sum1;
        l2 = l2 * c2 + sum2;
        const int j_begin = max(0, lo - tile);
        const int j_end = min(DIFF_TILE, pos - tile + 1);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int d = tid + c * DIFF_TILE;
            if (d < vdim) {
                float x1 = a1[c] * c1, x2 = a2[c] * c2;
                for (int jj = j_begin; jj < j_end; ++jj) {
                    const float v = to_f32<T>(cache[off_s[jj] + d]);
                    x1 += p1_s[jj] * v;
                    x2 += p2_s[jj] * v;
                }
                a1[c] = x1;
                a2[c] = x2;
            }
        }
        m1 = n1;
        m2 = n2;
        __syncthreads();                                  // p_s / off_s are rewritten by the next tile
    }
    float o[2], ss = 0.0f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        o[c] = (tid + c * DIFF_TILE < vdim) ? a1[c] / l1 - lambda * (a2[c] / l2) : 0.0f;
        ss += o[c] * o[c];
    }
    ss = block_sum(ss, scratch);
    const float f = out_scale / sqrtf(ss / (float)vdim + eps);
    T* dst = out + (long)t * out_ld + (long)h * vdim;
#pragma unroll
    for (int c = 0; c < 2; ++c)
        if (tid + c * DIFF_TILE < vdim) dst[tid + c * DIFF_TILE] = from_f32<T>(o[c] * f);
}

// q: [n_tokens, q_ld], head h's two (rotated) maps at columns [h * 2 dim, (h + 1) * 2 dim); out: [n_tokens, out_ld],
// head h at columns [h * vdim, (h + 1) * vdim).  window <= 0: all keys.
FL_API int fl_diff_attention_simt(const void* q, int dtype, long q_ld, void* out, long out_ld, const void* cache,
                                  long page_stride, int page_size, const int* block_table, int bt_stride,
                                  const int* tok_req, const int* positions, int n_tokens, int heads, int kv_heads,
                                  int dim, int vdim, int window, float scale, float lambda, float eps, float out_scale,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (vdim < 1 || vdim > 2 * DIFF_TILE || dim < 1 || dim > 4096 || heads > 65535 || heads % kv_heads)
        return (int)cudaErrorInvalidValue;
    const size_t smem = DIFF_TILE * (sizeof(long) + 2 * sizeof(float)) + (size_t)2 * dim * sizeof(float);
    dim3 grid(n_tokens, heads);
    FL_DISPATCH(dtype, T, return fl_launch(diff_attention_simt_kernel<T>, grid, dim3(DIFF_TILE), smem, stream,
                                           (const T*)q, q_ld, (T*)out, out_ld, (const T*)cache, page_stride, page_size,
                                           block_table, bt_stride, tok_req, positions, heads, kv_heads, dim, vdim,
                                           window, scale, lambda, eps, out_scale));
    return 0;
}
