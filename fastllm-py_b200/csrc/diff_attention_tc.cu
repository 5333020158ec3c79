// Differential attention over a paged cache on the tensor cores (bfloat16, mma.sync m16n8k16),
// softmax, difference and norm in float.
//
// A query head carries two maps (q1 | q2, DIFF_DIM each); a cache row holds a token's two key maps and
// its value (k1 | k2 | v, DIFF_VDIM the last).  Per head, with a_m = softmax(q_m . k_m * scale) V:
//     o = a_1 - lambda a_2;   out = o / sqrt(mean(o^2) + eps) * out_scale
//
// A CTA of eight warps (four per map, 16 rows each) takes 64 consecutive query rows of one request and one query
// head and walks the
// request's keys in blocks of 64, from the first key any of its rows may see to the last, through the
// block table: rows cached by earlier steps and the rows this step wrote are read alike, so a portion
// of a prompt is the same as a whole prompt, and a single decoded token is a tile of one row (warps
// without rows only help to load; steps of single tokens have a kernel of their own that splits the keys,
// diff_attention.cu, and the launcher can leave such requests out).  Key blocks start at multiples of 64 of the absolute position, so
// the partial maxima and sums a row goes through depend on the row's position only.  A block's rows
// (both key maps and the value: one piece of memory per token) come by cp.async into a two-stage ring
// while the block before is multiplied; both maps are multiplied against the same staged values, each
// by its own four warps with a running maximum and sum of its own (half the accumulators per thread,
// twice the warps an SM holds), and meet only in the epilogue: the second map's warps leave their
// normalised rows in shared memory, the first map's take the difference, sum the row's mean square over
// the four lanes that hold it and store.  Probabilities are rounded to bfloat16 only as
// the operand of P V.
//
// DIFF_DIM and DIFF_VDIM are compile-time constants, multiples of 16 up to 128.
#include "common.cuh"

#ifndef DIFF_DIM
#define DIFF_DIM 64
#endif
#ifndef DIFF_VDIM
#define DIFF_VDIM 128
#endif
#define DTC_BM 64
#define DTC_BN 64
#define DTC_THREADS 256
#define DTC_ROW (2 * DIFF_DIM + DIFF_VDIM)    // elements of a cache row
#define DTC_KP (DTC_ROW + 8)                  // padded pitches in shared memory: ldmatrix without bank conflicts
#define DTC_QP (2 * DIFF_DIM + 8)

static_assert(DIFF_DIM % 16 == 0 && DIFF_DIM >= 16 && DIFF_DIM <= 128, "DIFF_DIM: multiple of 16, at most 128");
static_assert(DIFF_VDIM % 16 == 0 && DIFF_VDIM >= 16 && DIFF_VDIM <= 128, "DIFF_VDIM: multiple of 16, at most 128");

__device__ __forceinline__ uint32_t dtc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void dtc_cp16(void* dst, const void* src, bool real) {
    const int bytes = real ? 16 : 0;                       // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dtc_smem(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void dtc_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void dtc_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void dtc_ldm(uint32_t* r, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(dtc_smem(p)));
}
__device__ __forceinline__ void dtc_ldm_t(uint32_t* r, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(dtc_smem(p)));
}
__device__ __forceinline__ void dtc_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t dtc_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float dtc_weight(float a, float b) { return (a == -CUDART_INF_F) ? 0.0f : exp2f(a - b); }

__global__ void __launch_bounds__(DTC_THREADS, 2) diff_attention_tc_kernel(
    const bf16* __restrict__ q, long q_ld, bf16* __restrict__ out, long out_ld, const bf16* __restrict__ cache,
    long page_stride, int page_size, int page_shift, const int* __restrict__ block_table, int bt_stride,
    const int* __restrict__ req_start, const int* __restrict__ req_ctx, const int* __restrict__ req_qlen,
    int n_requests, int include_single, int heads, int kv_heads, int window, float scale_log2e, float lambda, float eps,
    float out_scale) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) unsigned char dtc_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(dtc_raw);                       // [64][QP]
    bf16* Rs = Qs + DTC_BM * DTC_QP;                                   // [2 stages][64][KP]

    // which request and which 64-row tile of it this CTA serves (heaviest tiles first)
    int req = -1, tile = 0;
    {
        int acc = 0;
        for (int r = 0; r < n_requests; ++r) {
            const int ql = req_qlen[r];
            const int nt = (ql > 1 || include_single) ? (ql + DTC_BM - 1) / DTC_BM : 0;
            if ((int)blockIdx.x < acc + nt) { req = r; tile = nt - 1 - ((int)blockIdx.x - acc); break; }
            acc += nt;
        }
    }
    if (req < 0) return;
    const int h = blockIdx.y;
    const int kvh = h / (heads / kv_heads);
    const int q_len = req_qlen[req], ctx = req_ctx[req], row0 = tile * DTC_BM;
    const int tok0 = req_start[req] + row0;
    const int rows_here = min(DTC_BM, q_len - row0);
    const int pos_first = ctx + row0, pos_last = ctx + row0 + rows_here - 1;
    const int lo_tile = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int kb_begin = lo_tile / DTC_BN, kb_end = pos_last / DTC_BN + 1;
    const int* bt = block_table + (long)req * bt_stride;
    const int tid = threadIdx.x, lane = tid & 31;
    const int m = tid >> 7;                                            // this warp's map
    const int warp = (tid >> 5) & 3;                                   // which 16 rows of the tile
    const bool has_rows = warp * 16 < rows_here;                       // a warp without rows only loads

    constexpr int Q_CHUNKS = 2 * DIFF_DIM / 8, R_CHUNKS = DTC_ROW / 8;
    auto load_q = [&]() {
        for (int c = tid; c < DTC_BM * Q_CHUNKS; c += DTC_THREADS) {
            const int r = c / Q_CHUNKS, ch = c - r * Q_CHUNKS;
            const bool real = r < rows_here;
            const bf16* src = q + (long)(tok0 + (real ? r : 0)) * q_ld + (long)h * 2 * DIFF_DIM + ch * 8;
            dtc_cp16(Qs + r * DTC_QP + ch * 8, src, real);
        }
    };
    // Four threads per token row, a quarter of the row's chunks each: one page lookup per thread and block.
    auto load_rows = [&](int kb, int stage) {
        bf16* dst = Rs + stage * DTC_BN * DTC_KP;
        const int r = tid >> 2;
        const int j = kb * DTC_BN + r;
        const bool real = j >= lo_tile && j <= pos_last;
        long a = 0;
        if (real) {
            const int pg = page_shift >= 0 ? (j >> page_shift) : (j / page_size);
            const int off = page_shift >= 0 ? (j & (page_size - 1)) : (j - pg * page_size);
            a = (long)bt[pg] * page_stride + ((long)kvh * page_size + off) * DTC_ROW;
        }
        for (int ch = (tid & 3); ch < R_CHUNKS; ch += 4) dtc_cp16(dst + r * DTC_KP + ch * 8, cache + a + ch * 8, real);
    };

    float o_acc[DIFF_VDIM / 8][4];
#pragma unroll
    for (int i = 0; i < DIFF_VDIM / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.0f;
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F};
    float l_run[2] = {0.0f, 0.0f};
    const int g = lane >> 2, tq = lane & 3;
    const int pos_row[2] = {ctx + row0 + warp * 16 + g, ctx + row0 + warp * 16 + g + 8};

    load_q();
    load_rows(kb_begin, 0);
    dtc_commit();

    for (int kb = kb_begin; kb < kb_end; ++kb) {
        const int stage = (kb - kb_begin) & 1;
        if (kb + 1 < kb_end) {
            load_rows(kb + 1, stage ^ 1);
            dtc_commit();
            dtc_wait<1>();
        } else {
            dtc_wait<0>();
        }
        __syncthreads();
        const bf16* rt = Rs + stage * DTC_BN * DTC_KP;
        const int warp_pos_lo = ctx + row0 + warp * 16, warp_pos_hi = warp_pos_lo + 15;
        const bool all_seen = (kb * DTC_BN + DTC_BN - 1 <= warp_pos_lo) && (window <= 0 || kb * DTC_BN > warp_pos_hi - window);
        // a block none of this warp's rows can see (the tile's rows are 64 positions apart at most, a warp's 16)
        const bool none_seen = kb * DTC_BN > warp_pos_hi || (window > 0 && kb * DTC_BN + DTC_BN - 1 <= warp_pos_lo - window);
        if (has_rows && !none_seen) {
            {
                // ---- S = Q_m K_m^T for this warp's 16 rows and the block's 64 keys
                float s[DTC_BN / 8][4];
#pragma unroll
                for (int i = 0; i < DTC_BN / 8; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
#pragma unroll
                for (int ks = 0; ks < DIFF_DIM / 16; ++ks) {
                    uint32_t a[4];
                    dtc_ldm(a, Qs + (warp * 16 + (lane & 15)) * DTC_QP + m * DIFF_DIM + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int np = 0; np < DTC_BN / 16; ++np) {
                        uint32_t b[4];
                        dtc_ldm(b, rt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * DTC_KP + m * DIFF_DIM + ks * 16 +
                                       ((lane >> 3) & 1) * 8);
                        dtc_mma(s[2 * np], a, b[0], b[1]);
                        dtc_mma(s[2 * np + 1], a, b[2], b[3]);
                    }
                }
                // ---- scale, mask, running softmax (maxima and sums in units of log2)
                float corr[2];
                float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
                for (int nt = 0; nt < DTC_BN / 8; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        bool seen = true;
                        if (!all_seen) {
                            const int j = kb * DTC_BN + nt * 8 + 2 * tq + (e & 1);
                            const int pr = pos_row[e >> 1];
                            seen = j <= pr && (window <= 0 || j > pr - window);
                        }
                        const float v = seen ? s[nt][e] * scale_log2e : -CUDART_INF_F;
                        s[nt][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
                }
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                    const float m_new = fmaxf(m_run[r], mx[r]);
                    corr[r] = dtc_weight(m_run[r], m_new);
                    m_run[r] = m_new;
                    l_run[r] *= corr[r];
                }
#pragma unroll
                for (int nt = 0; nt < DTC_BN / 8; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float p = dtc_weight(s[nt][e], m_run[e >> 1]);
                        s[nt][e] = p;
                        l_run[e >> 1] += p;
                    }
                }
#pragma unroll
                for (int i = 0; i < DIFF_VDIM / 8; ++i) {
                    o_acc[i][0] *= corr[0];
                    o_acc[i][1] *= corr[0];
                    o_acc[i][2] *= corr[1];
                    o_acc[i][3] *= corr[1];
                }
                // ---- O_m += P_m V
#pragma unroll
                for (int kk = 0; kk < DTC_BN / 16; ++kk) {
                    uint32_t a[4];
                    a[0] = dtc_pack(s[2 * kk][0], s[2 * kk][1]);
                    a[1] = dtc_pack(s[2 * kk][2], s[2 * kk][3]);
                    a[2] = dtc_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                    a[3] = dtc_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                    for (int dp = 0; dp < DIFF_VDIM / 16; ++dp) {
                        uint32_t b[4];
                        dtc_ldm_t(b, rt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DTC_KP + 2 * DIFF_DIM + dp * 16 +
                                         (lane >> 4) * 8);
                        dtc_mma(o_acc[2 * dp], a, b[0], b[1]);
                        dtc_mma(o_acc[2 * dp + 1], a, b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();                                    // the stage is refilled two iterations on
    }
    // ---- the second map's warps leave their normalised rows (already times lambda) in shared memory, over the ring
    float* a2 = reinterpret_cast<float*>(Rs);                          // [64][VDIM]; the ring was read out before the barrier
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    if (m == 1 && has_rows) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float inv2 = lambda / l_run[r];
            float* dst = a2 + (warp * 16 + g + r * 8) * DIFF_VDIM + 2 * tq;
#pragma unroll
            for (int i = 0; i < DIFF_VDIM / 8; ++i)
                *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o_acc[i][2 * r] * inv2, o_acc[i][2 * r + 1] * inv2);
        }
    }
    __syncthreads();
    if (m == 1 || !has_rows) return;

    // ---- the first map's warps: the difference, the row's root mean square, store
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + g + r * 8;
        const float inv1 = 1.0f / l_run[r];
        const float* other = a2 + row * DIFF_VDIM + 2 * tq;
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < DIFF_VDIM / 8; ++i) {
            const float2 x = *reinterpret_cast<const float2*>(other + i * 8);
            const float o0 = o_acc[i][2 * r] * inv1 - x.x, o1 = o_acc[i][2 * r + 1] * inv1 - x.y;
            o_acc[i][2 * r] = o0;
            o_acc[i][2 * r + 1] = o1;
            ss += o0 * o0 + o1 * o1;
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        if (row >= rows_here) continue;
        const float f = out_scale / sqrtf(ss / (float)DIFF_VDIM + eps);
        bf16* dst = out + (long)(tok0 + row) * out_ld + (long)h * DIFF_VDIM + 2 * tq;
#pragma unroll
        for (int i = 0; i < DIFF_VDIM / 8; ++i) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(o_acc[i][2 * r] * f, o_acc[i][2 * r + 1] * f);
            *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = v;
        }
    }
}

FL_API int fl_diff_attention_tc_dim() { return DIFF_DIM; }
FL_API int fl_diff_attention_tc_vdim() { return DIFF_VDIM; }

// Every request r of the step with req_qlen[r] > 1 (or >= 1 with include_single) gets attention for its rows req_start[r] .. req_start[r] + req_qlen[r] - 1 at
// positions req_ctx[r] + i over its cached rows.  n_tokens bounds the number of 64-row tiles.
FL_API int fl_diff_attention_tc(const void* q, long q_ld, void* out, long out_ld, const void* cache, long page_stride,
                                int page_size, const int* block_table, int bt_stride, const int* req_start,
                                const int* req_ctx, const int* req_qlen, int n_requests, int n_tokens,
                                int include_single, int heads, int kv_heads, int window, float scale, float lambda, float eps, float out_scale,
                                cudaStream_t stream) {
    if (n_requests <= 0 || n_tokens <= 0) return 0;
    if (heads > 65535 || heads % kv_heads) return (int)cudaErrorInvalidValue;
    if ((q_ld % 8) || (out_ld % 2) || (page_stride % 8) || ((uintptr_t)q % 16) || ((uintptr_t)cache % 16) || ((uintptr_t)out % 4))
        return (int)cudaErrorMisalignedAddress;
    const size_t smem = ((size_t)DTC_BM * DTC_QP + 2 * (size_t)DTC_BN * DTC_KP) * sizeof(bf16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(diff_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    int page_shift = -1;
    if ((page_size & (page_size - 1)) == 0) {
        page_shift = 0;
        while ((1 << page_shift) < page_size) ++page_shift;
    }
    const int max_tiles = n_tokens / DTC_BM + n_requests;   // the sum of ceil(q_len / 64) is at most this
    dim3 grid(max_tiles, heads);
    return fl_launch(diff_attention_tc_kernel, grid, dim3(DTC_THREADS), smem, stream, (const bf16*)q, q_ld, (bf16*)out,
                     out_ld, (const bf16*)cache, page_stride, page_size, page_shift, block_table, bt_stride, req_start,
                     req_ctx, req_qlen, n_requests, include_single, heads, kv_heads, window, scale * 1.4426950408889634f,
                     lambda, eps, out_scale);
}
