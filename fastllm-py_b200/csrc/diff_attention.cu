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
//   diff_prep            per token: rotates the query maps in place; rotates the key maps into the
//                        token's cache rows and copies the values behind them
//   diff_attention_simt  per (token, query head): CUDA cores, any sizes, bfloat16 or true 32-bit;
//                        key tiles start at multiples of 128 of the absolute position, so every sum's
//                        order depends on the token's own position only (cuts and batches agree bit
//                        for bit)
//
//   diff_decode          single tokens with their keys split over blocks: per (token, key/value head, split of
//                        128 keys at a multiple of 128 of the absolute position) the maxima, sums and weighted
//                        values of both maps of every query head of the group, so that a cache row is read once
//                        for the group; diff_decode_merge adds the splits up and does the difference and the norm
//
// Scores, softmax, the difference and the norm are float.
#include "common.cuh"

#define DIFF_TILE 128

// One block per token.
template <typename T>
__global__ void __launch_bounds__(256) diff_prep_kernel(
    T* __restrict__ proj, long ld, int heads, int kv_heads, int dim, int vdim, int rot,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, const int* __restrict__ positions,
    const int* __restrict__ slots, T* __restrict__ cache, long page_stride, int page_size) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = rot >> 1;
    const long pos = positions[t];
    const float* cs = cos_table + pos * half;
    const float* sn = sin_table + pos * half;
    T* row = proj + (long)t * ld;
    for (int i = threadIdx.x; i < heads * 2 * half; i += blockDim.x) {        // every map of every query head, in place
        const int map = i / half, j = i - map * half;
        T* xm = row + (long)map * dim;
        const float a = to_f32<T>(xm[j]), b = to_f32<T>(xm[j + half]);
        xm[j] = from_f32<T>(a * cs[j] - b * sn[j]);
        xm[j + half] = from_f32<T>(b * cs[j] + a * sn[j]);
    }
    if (cache == nullptr) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const long page = slot / page_size;
    const int off = slot - (int)page * page_size;
    const int row_w = 2 * dim + vdim;
    T* dst = cache + page * page_stride + (long)off * row_w;                   // head g's row: + g * page_size * row_w
    const long head_stride = (long)page_size * row_w;
    const T* k = row + (long)heads * 2 * dim;
    const T* v = k + (long)kv_heads * 2 * dim;
    for (int i = threadIdx.x; i < kv_heads * 2 * half; i += blockDim.x) {
        const int map = i / half, j = i - map * half;                          // map = 2 g + (0 | 1)
        const T* km = k + (long)map * dim;
        T* dm = dst + (map >> 1) * head_stride + (map & 1) * dim;
        const float a = to_f32<T>(km[j]), b = to_f32<T>(km[j + half]);
        dm[j] = from_f32<T>(a * cs[j] - b * sn[j]);
        dm[j + half] = from_f32<T>(b * cs[j] + a * sn[j]);
    }
    const int rest = dim - rot;
    for (int i = threadIdx.x; i < kv_heads * 2 * rest; i += blockDim.x) {
        const int map = i / rest, j = rot + i - map * rest;
        dst[(map >> 1) * head_stride + (map & 1) * dim + j] = k[(long)map * dim + j];
    }
    for (int i = threadIdx.x; i < kv_heads * vdim; i += blockDim.x) {
        const int g = i / vdim, j = i - g * vdim;
        dst[g * head_stride + 2 * dim + j] = v[i];
    }
}

// proj: [n_tokens, ld] with columns q (heads x 2 x dim) | k (kv_heads x 2 x dim) | v (kv_heads x vdim);
// cache (one layer's pages) may be null: the queries only are turned then.
FL_API int fl_diff_prep(void* proj, int dtype, long ld, int n_tokens, int heads, int kv_heads, int dim, int vdim, int rot,
                        const float* cos_table, const float* sin_table, const int* positions, const int* slots,
                        void* cache, long page_stride, int page_size, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot < 0 || rot > dim || (rot & 1)) return (int)cudaErrorInvalidValue;
    FL_DISPATCH(dtype, T, return fl_launch(diff_prep_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (T*)proj, ld, heads,
                                           kv_heads, dim, vdim, rot, cos_table, sin_table, positions, slots, (T*)cache,
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

// ------------------------------------------------------------------ single tokens, keys split over blocks
#define DIFF_SPLIT 128           // keys of a split: one per thread

__device__ __forceinline__ void load8(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

// GROUP: query heads per key/value head, rounded up to a power of two (at most 8); pair hm = 2 * head in group + map.
// partial: [n_decode][heads][2 maps][n_splits][vdim + 2] floats: maximum, sum, weighted values.
template <typename T, int GROUP>
__global__ void __launch_bounds__(DIFF_SPLIT) diff_decode_kernel(
    const T* __restrict__ q, long q_ld, const T* __restrict__ cache, long page_stride, int page_size,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tok_req, const int* __restrict__ positions,
    const int* __restrict__ decode_tokens, float* __restrict__ partial, int n_splits, int heads, int kv_heads, int dim,
    int vdim, int window, float scale, int vec8) {
    pdl_wait();
    pdl_trigger();
    constexpr int GM = 2 * GROUP;
    extern __shared__ __align__(16) unsigned char dec_smem[];
    long* off_s = reinterpret_cast<long*>(dec_smem);                  // [SPLIT] element offset of each row's value part
    float* p_s = reinterpret_cast<float*>(off_s + DIFF_SPLIT);        // [SPLIT][GM] numerators
    float* red_s = p_s + DIFF_SPLIT * GM;                             // [4 warps][GM]
    float* q_s = red_s + 4 * GM;                                      // [GM][dim]
    const int t = decode_tokens[blockIdx.x], g = blockIdx.y, split = blockIdx.z, tid = threadIdx.x;
    const int group = heads / kv_heads;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int first = (lo / DIFF_SPLIT + split) * DIFF_SPLIT;
    const int row_w = 2 * dim + vdim;
    float* out = partial + ((((long)blockIdx.x * heads + (long)g * group) * 2) * n_splits + split) * (vdim + 2);
    const long hm_stride = (long)n_splits * (vdim + 2);               // from one (head, map) pair to the next
    if (first > pos) {                                                // nothing of this token in the split
        for (int hm = tid; hm < 2 * group; hm += DIFF_SPLIT) {
            out[hm * hm_stride] = -CUDART_INF_F;
            out[hm * hm_stride + 1] = 0.0f;
        }
        return;
    }
    for (int i = tid; i < 2 * group * dim; i += DIFF_SPLIT)
        q_s[i] = to_f32<T>(q[(long)t * q_ld + (long)g * group * 2 * dim + i]);
    __syncthreads();
    const int* bt = block_table + (long)tok_req[t] * bt_stride;
    const int j = first + tid;
    const bool valid = j >= lo && j <= pos;
    float s[GM];
#pragma unroll
    for (int hm = 0; hm < GM; ++hm) s[hm] = 0.0f;
    if (valid) {
        const long off = (long)bt[j / page_size] * page_stride + ((long)g * page_size + j % page_size) * row_w;
        off_s[tid] = off + 2 * dim;
        const T* kp = cache + off;
        if (vec8) {                                                   // eight elements of both maps per load
            for (int d = 0; d < dim; d += 8) {
                float k1[8], k2[8];
                load8(kp + d, k1);
                load8(kp + dim + d, k2);
#pragma unroll
                for (int e = 0; e < 8; ++e)
#pragma unroll
                    for (int hh = 0; hh < GROUP; ++hh)
                        if (hh < group) {
                            s[2 * hh] += q_s[(2 * hh) * dim + d + e] * k1[e];
                            s[2 * hh + 1] += q_s[(2 * hh + 1) * dim + d + e] * k2[e];
                        }
            }
        } else {
            for (int d = 0; d < dim; ++d) {
                const float k1 = to_f32<T>(kp[d]), k2 = to_f32<T>(kp[dim + d]);
#pragma unroll
                for (int hh = 0; hh < GROUP; ++hh)
                    if (hh < group) {
                        s[2 * hh] += q_s[(2 * hh) * dim + d] * k1;
                        s[2 * hh + 1] += q_s[(2 * hh + 1) * dim + d] * k2;
                    }
            }
        }
    }
    const int warp = tid >> 5, lane = tid & 31;
    float m[GM];
#pragma unroll
    for (int hm = 0; hm < GM; ++hm) {
        s[hm] = valid ? s[hm] * scale : -CUDART_INF_F;
        const float w = warp_max(s[hm]);
        if (lane == 0) red_s[warp * GM + hm] = w;
    }
    __syncthreads();
#pragma unroll
    for (int hm = 0; hm < GM; ++hm) {
        m[hm] = fmaxf(fmaxf(red_s[hm], red_s[GM + hm]), fmaxf(red_s[2 * GM + hm], red_s[3 * GM + hm]));
        const float p = valid ? expf(s[hm] - m[hm]) : 0.0f;          // (some key of the split is valid: m is finite)
        p_s[tid * GM + hm] = p;
        s[hm] = warp_sum(p);
    }
    __syncthreads();                                                  // red_s was read; p_s and off_s are written
#pragma unroll
    for (int hm = 0; hm < GM; ++hm)
        if (lane == 0) red_s[warp * GM + hm] = s[hm];
    __syncthreads();
#pragma unroll
    for (int hm = 0; hm < GM; ++hm)
        if (tid == hm && hm < 2 * group) {                            // (m is the same in every thread)
            out[hm * hm_stride] = m[hm];
            out[hm * hm_stride + 1] = red_s[hm] + red_s[GM + hm] + red_s[2 * GM + hm] + red_s[3 * GM + hm];
        }
    const int j_begin = max(0, lo - first), j_end = min(DIFF_SPLIT, pos - first + 1);
    for (int d = tid; d < vdim; d += DIFF_SPLIT) {
        float acc[GM];
#pragma unroll
        for (int hm = 0; hm < GM; ++hm) acc[hm] = 0.0f;
#pragma unroll 8
        for (int jj = j_begin; jj < j_end; ++jj) {
            const float v = to_f32<T>(cache[off_s[jj] + d]);
#pragma unroll
            for (int hm = 0; hm < GM; ++hm) acc[hm] += p_s[jj * GM + hm] * v;
        }
#pragma unroll
        for (int hm = 0; hm < GM; ++hm)
            if (hm < 2 * group) out[hm * hm_stride + 2 + d] = acc[hm];
    }
}

// One block per (token, query head): both maps' splits added up, the difference, the norm.
template <typename T>
__global__ void __launch_bounds__(128) diff_decode_merge_kernel(const float* __restrict__ partial, int n_splits,
                                                                const int* __restrict__ decode_tokens, T* __restrict__ out,
                                                                long out_ld, int heads, int vdim, float lambda, float eps,
                                                                float out_scale) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[32];
    const int h = blockIdx.y, tid = threadIdx.x;
    const float* base = partial + (((long)blockIdx.x * heads + h) * 2) * n_splits * (vdim + 2);
    float top[2] = {-CUDART_INF_F, -CUDART_INF_F}, sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
        const float* pm = base + (long)mp * n_splits * (vdim + 2);
        for (int s = 0; s < n_splits; ++s) top[mp] = fmaxf(top[mp], pm[(long)s * (vdim + 2)]);
        for (int s = 0; s < n_splits; ++s) {
            const float ms = pm[(long)s * (vdim + 2)];
            if (ms != -CUDART_INF_F) sum[mp] += pm[(long)s * (vdim + 2) + 1] * expf(ms - top[mp]);
        }
    }
    float o[2] = {0.0f, 0.0f}, ss = 0.0f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int d = tid + c * 128;
        if (d >= vdim) continue;
        float a[2] = {0.0f, 0.0f};
#pragma unroll
        for (int mp = 0; mp < 2; ++mp) {
            const float* pm = base + (long)mp * n_splits * (vdim + 2);
            for (int s = 0; s < n_splits; ++s) {
                const float ms = pm[(long)s * (vdim + 2)];
                if (ms != -CUDART_INF_F) a[mp] += pm[(long)s * (vdim + 2) + 2 + d] * expf(ms - top[mp]);
            }
        }
        o[c] = a[0] / sum[0] - lambda * (a[1] / sum[1]);
        ss += o[c] * o[c];
    }
    ss = block_sum(ss, scratch);
    const float f = out_scale / sqrtf(ss / (float)vdim + eps);
    T* dst = out + (long)decode_tokens[blockIdx.x] * out_ld + (long)h * vdim;
#pragma unroll
    for (int c = 0; c < 2; ++c)
        if (tid + c * 128 < vdim) dst[tid + c * 128] = from_f32<T>(o[c] * f);
}

// Whether the split-key kernels take a layer of these sizes.
FL_API int fl_diff_decode_takes(int heads, int kv_heads, int dim, int vdim) {
    const int group = kv_heads > 0 && heads % kv_heads == 0 ? heads / kv_heads : 0;
    return group >= 1 && group <= 8 && vdim >= 1 && vdim <= 256 && dim >= 1 &&
           (size_t)DIFF_SPLIT * (sizeof(long) + 16 * sizeof(float)) + (size_t)(64 + 16 * dim) * sizeof(float) <= 48 * 1024;
}

// The rows `decode_tokens` (n_decode of them, each the single token of its request) of q get attention over their
// requests' cache rows; n_splits must reach every token's last key: (longest visible span - 1) / 128 + 2 does.
// partial: n_decode * heads * 2 * n_splits * (vdim + 2) floats.
FL_API int fl_diff_decode(const void* q, int dtype, long q_ld, void* out, long out_ld, const void* cache, long page_stride,
                          int page_size, const int* block_table, int bt_stride, const int* tok_req, const int* positions,
                          const int* decode_tokens, int n_decode, float* partial, int n_splits, int heads, int kv_heads,
                          int dim, int vdim, int window, float scale, float lambda, float eps, float out_scale,
                          cudaStream_t stream) {
    if (n_decode <= 0) return 0;
    if (!fl_diff_decode_takes(heads, kv_heads, dim, vdim) || n_splits < 1 || n_splits > 65535 || kv_heads > 65535)
        return (int)cudaErrorInvalidValue;
    const int group = heads / kv_heads;
    const int gp = group <= 1 ? 1 : group <= 2 ? 2 : group <= 4 ? 4 : 8;
    const size_t smem = (size_t)DIFF_SPLIT * (sizeof(long) + 2 * gp * sizeof(float)) + (size_t)(8 * gp + 2 * gp * dim) * sizeof(float);
    dim3 grid(n_decode, kv_heads, n_splits);
    // (rows start 16 bytes aligned when the row and page sizes are multiples of 8 elements and the pool is aligned)
    const int vec8 = dim % 8 == 0 && vdim % 8 == 0 && page_stride % 8 == 0 && ((uintptr_t)cache % 32) == 0;
    int rc = 0;
#define FL_DIFF_DECODE(G)                                                                                            \
    FL_DISPATCH(dtype, T, rc = fl_launch(diff_decode_kernel<T, G>, grid, dim3(DIFF_SPLIT), smem, stream, (const T*)q, \
                                         q_ld, (const T*)cache, page_stride, page_size, block_table, bt_stride,      \
                                         tok_req, positions, decode_tokens, partial, n_splits, heads, kv_heads, dim, \
                                         vdim, window, scale, vec8))
    if (gp == 1) { FL_DIFF_DECODE(1); }
    else if (gp == 2) { FL_DIFF_DECODE(2); }
    else if (gp == 4) { FL_DIFF_DECODE(4); }
    else { FL_DIFF_DECODE(8); }
#undef FL_DIFF_DECODE
    if (rc) return rc;
    FL_DISPATCH(dtype, T, return fl_launch(diff_decode_merge_kernel<T>, dim3(n_decode, heads), dim3(128), 0, stream,
                                           (const float*)partial, n_splits, decode_tokens, (T*)out, out_ld, heads, vdim,
                                           lambda, eps, out_scale));
    return 0;
}
