// Latent attention on tensor cores (bfloat16 mma.sync m16n8k16), one build per (LAT_RANK, LAT_ROT).
//
// The same computation as latent_attention.cu's kernel: per token and head, softmax over the visible
// cache rows of q~ . [c | rotated part] * scale, then the weighted sum of the rows' first LAT_RANK
// elements.  All heads share a token's rows, so a block takes one token and 16 heads as the 16 rows of
// the MMA's A operand: decode steps use the tensor cores at full width, and a cache row that a block
// stages in shared memory serves 16 heads.
//
// A block has 4 warps and walks the keys in tiles of 32 (aligned to absolute positions), two tiles in
// flight through cp.async.  Per tile: warp w computes the scores of keys 8w..8w+7 (q~ from shared
// memory, the rows as the col-major B operand), the row maxima and sums cross the warps through shared
// memory, the probabilities go to shared memory in bfloat16, and warp w accumulates its quarter of the
// value columns over all 32 keys (the staged rows read through ldmatrix.trans).  Scores, maxima, sums and
// the output accumulator are float; the accumulator is rescaled at every tile.
#include "common.cuh"

#ifndef LAT_RANK
#error "build with -DLAT_RANK=<latent size> -DLAT_ROT=<rotated key size>"
#endif
#define LT_WIDTH (LAT_RANK + LAT_ROT)
#define LT_PITCH (LT_WIDTH + 8)          // bfloat16 elements between staged rows (ldmatrix without bank conflicts)
#define LT_KEYS 32
#define LT_WARPS 4
#define LT_VCOLS (LAT_RANK / LT_WARPS)   // value columns of a warp
#define LT_NT (LT_VCOLS / 8)
#define LT_PPITCH (LT_KEYS + 8)
static_assert(LAT_RANK % 32 == 0 && LT_WIDTH % 16 == 0, "latent size must be a multiple of 32, row width of 16");

__device__ __forceinline__ void lt_cp16(void* smem, const void* gmem, int bytes) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes));
}

template <typename TO>
__global__ void __launch_bounds__(LT_WARPS * 32) latent_attention_tc_kernel(
    const bf16* __restrict__ q, long q_ld, TO* __restrict__ out, long out_ld, const bf16* __restrict__ cache,
    int page_size, const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tok_req,
    const int* __restrict__ positions, int heads, int window, float scale, int split_keys, float* __restrict__ partial) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) unsigned char lt_smem[];
    bf16* q_s = reinterpret_cast<bf16*>(lt_smem);                         // [16][LT_PITCH]
    bf16* k_s = q_s + 16 * LT_PITCH;                                      // [2][LT_KEYS][LT_PITCH]
    bf16* p_s = k_s + 2 * LT_KEYS * LT_PITCH;                             // [16][LT_PPITCH]
    float* red_max = reinterpret_cast<float*>(p_s + 16 * LT_PPITCH);      // [LT_WARPS][16]
    float* red_sum = red_max + LT_WARPS * 16;                             // [LT_WARPS][16]
    const int t = blockIdx.x, head0 = blockIdx.y * 16;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* bt = block_table + (long)tok_req[t] * bt_stride;

    auto stage = [&](int buf, int tile) {
        bf16* dst = k_s + (long)buf * LT_KEYS * LT_PITCH;
        constexpr int CHUNKS = LT_WIDTH / 8;
        for (int c = tid; c < LT_KEYS * CHUNKS; c += LT_WARPS * 32) {
            const int r = c / CHUNKS, piece = c % CHUNKS;
            const int j = tile + r;
            const bool valid = j >= lo && j <= pos;
            const bf16* src = cache;
            if (valid) src = cache + ((long)bt[j / page_size] * page_size + j % page_size) * LT_WIDTH + piece * 8;
            lt_cp16(dst + r * LT_PITCH + piece * 8, src, valid ? 16 : 0);     // rows out of sight are zeros
        }
        asm volatile("cp.async.commit_group;");
    };
    // with split_keys (a multiple of LT_KEYS) the block takes only the keys of split blockIdx.z, counted from
    // the multiple of split_keys at or below the first visible key, and leaves (accumulator, maximum, sum)
    // in `partial` for the merge kernel; the splits' borders depend on the token's own position only
    int first_tile = (lo / LT_KEYS) * LT_KEYS, last = pos;
    if (split_keys > 0) {
        first_tile = (lo / split_keys + (int)blockIdx.z) * split_keys;
        last = min(pos, first_tile + split_keys - 1);
        first_tile = max(first_tile, (lo / LT_KEYS) * LT_KEYS);      // (no tile wholly out of sight: its maximum would be -inf)
    }
    float* part_row = nullptr;
    if (split_keys > 0) {
        part_row = partial + (((long)t * heads) * gridDim.z + blockIdx.z) * (LAT_RANK + 2);     // + head * gridDim.z * (rank + 2)
        if (first_tile > pos) {                              // nothing of this split is in sight
            for (int r = tid; r < 16 && head0 + r < heads; r += LT_WARPS * 32) {
                float* pr = part_row + (long)(head0 + r) * gridDim.z * (LAT_RANK + 2);
                pr[LAT_RANK] = -CUDART_INF_F;
                pr[LAT_RANK + 1] = 0.0f;
            }
            return;
        }
    }
    stage(0, first_tile);
    for (int c = tid; c < 16 * (LT_WIDTH / 8); c += LT_WARPS * 32) {     // the 16 heads' q~
        const int r = c / (LT_WIDTH / 8), piece = c % (LT_WIDTH / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (head0 + r < heads) v = *reinterpret_cast<const uint4*>(q + (long)t * q_ld + (long)(head0 + r) * LT_WIDTH + piece * 8);
        *reinterpret_cast<uint4*>(q_s + r * LT_PITCH + piece * 8) = v;
    }
    float acc[LT_NT][4];
#pragma unroll
    for (int n = 0; n < LT_NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.0f, 0.0f};   // rows lane / 4 and lane / 4 + 8
    const int row0 = lane >> 2;
    int buf = 0;
    for (int tile = first_tile; tile <= last; tile += LT_KEYS, buf ^= 1) {
        if (tile + LT_KEYS <= last) {
            stage(buf ^ 1, tile + LT_KEYS);
            asm volatile("cp.async.wait_group 1;");
        } else {
            asm volatile("cp.async.wait_group 0;");
        }
        __syncthreads();
        const bf16* ks = k_s + (long)buf * LT_KEYS * LT_PITCH;
        // ---- scores of this warp's 8 keys
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
        for (int kk = 0; kk < LT_WIDTH; kk += 16) {
            unsigned a[4], b[2];
            const unsigned qa = (unsigned)__cvta_generic_to_shared(q_s + (lane & 15) * LT_PITCH + kk + (lane >> 4) * 8);
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(qa));
            const unsigned ka = (unsigned)__cvta_generic_to_shared(ks + (warp * 8 + (lane & 7)) * LT_PITCH + kk + ((lane >> 3) & 1) * 8);
            asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(b[0]), "=r"(b[1]) : "r"(ka));
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(s[0]), "+f"(s[1]), "+f"(s[2]), "+f"(s[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
        }
        const int j0 = tile + warp * 8 + (lane & 3) * 2;
        float mx[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int j = j0 + c;
                s[h * 2 + c] = (j >= lo && j <= pos) ? s[h * 2 + c] * scale : -CUDART_INF_F;
            }
            mx[h] = fmaxf(s[h * 2], s[h * 2 + 1]);
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        }
        if ((lane & 3) == 0) {
            red_max[warp * 16 + row0] = mx[0];
            red_max[warp * 16 + row0 + 8] = mx[1];
        }
        __syncthreads();
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = row0 + h * 8;
            float m_new = m_run[h];
#pragma unroll
            for (int w = 0; w < LT_WARPS; ++w) m_new = fmaxf(m_new, red_max[w * 16 + r]);
            corr[h] = expf(m_run[h] - m_new);               // 0 at the first tile
            m_run[h] = m_new;
            const float p0 = expf(s[h * 2] - m_new), p1 = expf(s[h * 2 + 1] - m_new);   // exp(-inf) = 0 out of sight
            float sum = p0 + p1;
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((lane & 3) == 0) red_sum[warp * 16 + r] = sum;
            *reinterpret_cast<__nv_bfloat162*>(p_s + r * LT_PPITCH + warp * 8 + (lane & 3) * 2) = __floats2bfloat162_rn(p0, p1);
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < LT_WARPS; ++w) sum += red_sum[w * 16 + row0 + h * 8];
            l_run[h] = l_run[h] * corr[h] + sum;
        }
#pragma unroll
        for (int n = 0; n < LT_NT; ++n) {
            acc[n][0] *= corr[0]; acc[n][1] *= corr[0];
            acc[n][2] *= corr[1]; acc[n][3] *= corr[1];
        }
        // ---- this warp's value columns over the tile's 32 keys
#pragma unroll
        for (int kk = 0; kk < LT_KEYS; kk += 16) {
            unsigned a[4];
            const unsigned pa = (unsigned)__cvta_generic_to_shared(p_s + (lane & 15) * LT_PPITCH + kk + (lane >> 4) * 8);
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(pa));
#pragma unroll
            for (int n = 0; n < LT_NT; ++n) {
                unsigned b[2];
                const unsigned va = (unsigned)__cvta_generic_to_shared(ks + (kk + (lane & 15)) * LT_PITCH + warp * LT_VCOLS + n * 8);
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b[0]), "=r"(b[1]) : "r"(va));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(acc[n][0]), "+f"(acc[n][1]), "+f"(acc[n][2]), "+f"(acc[n][3])
                             : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
            }
        }
        __syncthreads();                                     // the tile, p_s and the reductions are rewritten next
    }
    if (split_keys > 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int head = head0 + row0 + h * 8;
            if (head >= heads) continue;
            float* pr = part_row + (long)head * gridDim.z * (LAT_RANK + 2);
            float* o = pr + warp * LT_VCOLS + (lane & 3) * 2;
#pragma unroll
            for (int n = 0; n < LT_NT; ++n) {
                o[n * 8] = acc[n][h * 2];
                o[n * 8 + 1] = acc[n][h * 2 + 1];
            }
            if (warp == 0 && (lane & 3) == 0) {
                pr[LAT_RANK] = m_run[h];
                pr[LAT_RANK + 1] = l_run[h];
            }
        }
        return;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int head = head0 + row0 + h * 8;
        if (head >= heads) continue;
        TO* o = out + (long)t * out_ld + (long)head * LAT_RANK + warp * LT_VCOLS + (lane & 3) * 2;
        const float inv = 1.0f / l_run[h];
#pragma unroll
        for (int n = 0; n < LT_NT; ++n) {
            o[n * 8] = from_f32<TO>(acc[n][h * 2] * inv);
            o[n * 8 + 1] = from_f32<TO>(acc[n][h * 2 + 1] * inv);
        }
    }
}

// out[t, head] = sum_z acc_z e^(m_z - M) / sum_z l_z e^(m_z - M), splits in order; one block per (token, head).
template <typename TO>
__global__ void __launch_bounds__(128) latent_merge_kernel(const float* __restrict__ partial, TO* __restrict__ out,
                                                           long out_ld, int heads, int n_splits) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, head = blockIdx.y;
    const float* pr = partial + ((long)t * heads + head) * n_splits * (LAT_RANK + 2);
    float mx = -CUDART_INF_F;
    for (int z = 0; z < n_splits; ++z) mx = fmaxf(mx, pr[(long)z * (LAT_RANK + 2) + LAT_RANK]);
    float l = 0.0f;
    for (int z = 0; z < n_splits; ++z) {
        const float* p = pr + (long)z * (LAT_RANK + 2);
        if (p[LAT_RANK + 1] > 0.0f) l += p[LAT_RANK + 1] * expf(p[LAT_RANK] - mx);
    }
    for (int c = threadIdx.x; c < LAT_RANK; c += blockDim.x) {
        float sum = 0.0f;
        for (int z = 0; z < n_splits; ++z) {
            const float* p = pr + (long)z * (LAT_RANK + 2);
            if (p[LAT_RANK + 1] > 0.0f) sum += p[c] * expf(p[LAT_RANK] - mx);
        }
        out[(long)t * out_ld + (long)head * LAT_RANK + c] = from_f32<TO>(sum / l);
    }
}

FL_API int fl_latent_attention_tc_rank() { return LAT_RANK; }
FL_API int fl_latent_attention_tc_rot() { return LAT_ROT; }

// q: bfloat16 [n_tokens, heads x (rank + rot)], rows 16-byte aligned; out: float or bfloat16 [n_tokens, heads x rank];
// cache: bfloat16 [pages][page_size][rank + rot].  window <= 0: all earlier tokens.
// split_keys > 0 (a multiple of 32): the keys are shared out over n_splits blocks per token (decode steps,
// where tokens are too few to fill the GPU); `partial` then holds n_tokens * heads * n_splits * (rank + 2)
// floats and a merge kernel follows.  n_splits must reach the last key of every token:
// (longest visible span - 1) / split_keys + 2 does.
FL_API int fl_latent_attention_tc(const void* q, long q_ld, void* out, int out_dtype, long out_ld, const void* cache, int page_size,
                                  const int* block_table, int bt_stride, const int* tok_req, const int* positions,
                                  int n_tokens, int heads, int window, float scale, int split_keys, int n_splits,
                                  float* partial, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (split_keys < 0 || split_keys % LT_KEYS || (split_keys > 0 && (n_splits < 1 || n_splits > 65535 || partial == nullptr)))
        return (int)cudaErrorInvalidValue;
    if (((uintptr_t)q % 16) || (q_ld % 8) || ((uintptr_t)cache % 16) || (heads + 15) / 16 > 65535)
        return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)(16 * LT_PITCH + 2 * LT_KEYS * LT_PITCH + 16 * LT_PPITCH) * sizeof(bf16) +
                        2 * LT_WARPS * 16 * sizeof(float);
    static bool raised = false;
    if (!raised && smem > 48 * 1024) {
        cudaError_t rc = cudaFuncSetAttribute(latent_attention_tc_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (rc == cudaSuccess)
            rc = cudaFuncSetAttribute(latent_attention_tc_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (rc != cudaSuccess) return (int)rc;
        raised = true;
    }
    int rc = 0;
    FL_DISPATCH(out_dtype, TO,
        rc = fl_launch(latent_attention_tc_kernel<TO>, dim3(n_tokens, (heads + 15) / 16, split_keys > 0 ? n_splits : 1),
                       dim3(LT_WARPS * 32), smem, stream, (const bf16*)q, q_ld, (TO*)out, out_ld, (const bf16*)cache,
                       page_size, block_table, bt_stride, tok_req, positions, heads, window, scale, split_keys, partial));
    if (rc || split_keys == 0) return rc;
    FL_DISPATCH(out_dtype, TO,
        return fl_launch(latent_merge_kernel<TO>, dim3(n_tokens, heads), dim3(128), 0, stream, (const float*)partial,
                         (TO*)out, out_ld, heads, n_splits));
    return 0;
}
