// Paged attention with mixed heads for prompt portions on the tensor cores (bfloat16 storage).
// Compiled per (key size, value size): -DRV_D=<d> -DRV_DV=<dv>, multiples of 16.
//
// The same function as attention_mixed.cu.  A block owns 16 query tokens of one request and
// ALL heads of them (H a multiple of 8, at most 32; 16 H threads), because the softmax of a head
// needs every head's scores.  Per tile of 32 keys, aligned to absolute position 0:
//   1. keys and values of the tile come from the pages into shared memory (16-byte cp.async);
//      the next tile's keys are requested as soon as this tile's scores are formed and its
//      values as soon as this tile's are used, so both travel behind the arithmetic;
//   2. warp w forms the raw scores of heads 2w, 2w+1: S_g = scale * Q_g K^T (mma.sync m16n8k16,
//      float32 accumulators; the block's query rows stay in shared memory) -> shared memory,
//      float32;
//   3. mixing, mask and running softmax in float32 on the CUDA cores: a thread owns 4
//      neighbouring keys of one query token for 8 heads, s'_h = sum_g M[h, g] s_g as 16 packed
//      multiply-adds (fma.rn.f32x2) per five 16-byte shared-memory loads; scores are kept in
//      units of log 2, so the exponentials are exp2; maxima and sums over a row by shuffles among the 8
//      lanes that share the token; once every thread has read its scores, P takes their place
//      in shared memory as bfloat16 (the row sum adds the rounded values);
//   4. warp w rescales and extends O_h += P_h V of its two heads (V by ldmatrix.trans).
// The sink enters as the initial maximum with a sum of 1.  The epilogue divides by the sum,
// multiplies by sigmoid(gate) and writes bfloat16.
// A launch with too few blocks for the GPU (one prompt of a few thousand tokens: the last blocks
// of a prompt walk twice the average number of tiles) shares every block's keys out over several
// blocks, one per stretch of positions aligned to absolute position 0; they leave maxima, sums
// and unnormalised values in a scratch buffer, and the merge kernel of attention_mixed.cu puts a
// token's stretches together in order, adds the sink once, divides and gates.
// Work per (query, key) pair: 2 H (d + dv) tensor-core FLOPs and 2 H^2 float32 FLOPs for the
// mixing, which the tensor cores cannot take in float32; from 16 heads on the mixing is the
// longer part.
#include "common.cuh"

#ifndef RV_D
#error "compile with -DRV_D=<key size> -DRV_DV=<value size>"
#endif
#if RV_D % 16 != 0 || RV_DV % 16 != 0 || RV_D > 256 || RV_DV > 256
#error "RV_D and RV_DV must be multiples of 16, at most 256"
#endif

#define AM_KT 32
#define AM_QT 16
#define AM_LOG2E 1.4426950408889634f
#define AM_LN2 0.6931471805599453f
#define AM_SS 40          // float32 score row: 32 + 8 (conflict-free fragment stores)
#define AM_PS 40          // bfloat16 probability row: 32 + 8

typedef __nv_bfloat16 bf16;

#define AM_CAT2(a, b, c) a##b##_##c
#define AM_CAT(a, b, c) AM_CAT2(a, b, c)
#define AM_NAME(base) AM_CAT(base, RV_D, RV_DV)

static thread_local char g_am_error[256] = "";
extern "C" const char* AM_NAME(rv_attention_mixed_mma_last_error_d)() { return g_am_error; }
#define AM_FAIL(...)                                         \
    do {                                                     \
        snprintf(g_am_error, sizeof(g_am_error), __VA_ARGS__); \
        return 1;                                            \
    } while (0)

__device__ __forceinline__ void am_cp_async_16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zeroed
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void am_ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void am_ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
// two float32 multiply-adds in one instruction: c = a * b + c on both halves
__device__ __forceinline__ void am_fma2(unsigned long long& c, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c) : "l"(a), "l"(b));
}
__device__ __forceinline__ void am_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Up to 16 heads a block has 256 threads and two blocks share an SM (one's products run beside
// the other's mixing); above, 512 threads and one block.  128 registers either way.
template <int MAXT>
__global__ void __launch_bounds__(MAXT, MAXT == 256 ? 2 : 1)
attention_mixed_mma_kernel(const bf16* __restrict__ rows, int row_stride, int gate_off,
                           const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                           const int* __restrict__ block_table, int max_blocks,
                           const int* __restrict__ q_start, const int* __restrict__ ctx_lens,
                           bf16* __restrict__ out, int first_req, int H, int G, int page_size,
                           float scale, int window, int chunk, const float* __restrict__ mix,
                           const float* __restrict__ sinks, float* __restrict__ scratch, int stretch,
                           int first_token) {
    constexpr int D = RV_D, DV = RV_DV;
    rv_pdl_launch_dependents();
    const int r = first_req + blockIdx.y;
    const int q0 = q_start[r], q_len = q_start[r + 1] - q0;
    const int clen = ctx_lens[r];
    const int t_first = blockIdx.x * AM_QT;                  // first query token of the block
    if (clen == 0 || t_first >= q_len) return;
    const int KS = G * D + 8, VS = G * DV + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Ks = (bf16*)smem_raw;                              // [KT][KS]
    bf16* Vs = Ks + AM_KT * KS;                              // [KT][VS]
    float* S = (float*)(Vs + AM_KT * VS);                    // [H][QT][SS]
    bf16* P = (bf16*)S;                                      // [H][QT][PS]: takes S's place once every score is read
    const int QS = H * D + 8;
    bf16* Qs = (bf16*)(S + (size_t)H * AM_QT * AM_SS);       // [QT][QS]
    float* Tt = (float*)(Qs + AM_QT * QS);                   // [H][H][2]: Tt[g][h] = (mix[h][g], mix[h][g])
    float* alpha_s = Tt + 2 * H * H;                         // [H][QT]
    float* l_s = alpha_s + H * AM_QT;                        // [H][QT] running sums
    float* m_s = l_s + H * AM_QT;                            // [H][QT] running maxima
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hpg = H / G;
    const float scale2 = scale * AM_LOG2E;                   // scores are kept in units of log 2: exponentials are exp2
    for (int i = tid; i < H * H; i += blockDim.x) {
        const int g = i / H, h = i - g * H;
        const float m = mix ? mix[h * H + g] : (g == h ? 1.f : 0.f);
        Tt[2 * i] = m;                                       // both halves of a packed multiply-add
        Tt[2 * i + 1] = m;
    }
    const int p_first = clen - q_len + t_first;              // position of the block's first query
    const int n_q = min(AM_QT, q_len - t_first);
    // what the mixing thread owns: 8 heads, one query token, 4 neighbouring keys of a tile
    const int hb = tid >> 7, mq = (tid & 127) >> 3, kg = tid & 7;
    const int mp = p_first + mq;                             // its query's position
    int mlo = 0;
    if (window > 0) mlo = max(mlo, mp - window + 1);
    if (chunk > 0) mlo = max(mlo, mp / chunk * chunk);
    const bool mq_live = mq < n_q;
    // running maximum and sum of a (head, token): read by the 8 lanes that share the token,
    // written by the first of them; a tile touches each once, between two block barriers
    if (kg == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            m_s[(hb * 8 + j) * AM_QT + mq] = (sinks && !scratch) ? sinks[hb * 8 + j] * AM_LOG2E : -INFINITY;
            l_s[(hb * 8 + j) * AM_QT + mq] = (sinks && !scratch) ? 1.f : 0.f;
        }
    }
    int lo_first = 0;                                        // lowest key any query of the block sees
    if (window > 0) lo_first = max(lo_first, p_first - window + 1);
    if (chunk > 0) lo_first = max(lo_first, p_first / chunk * chunk);
    int p_last = p_first + n_q - 1;
    if (scratch) {
        // a launch that shares a block's keys out: this block takes the blockIdx.z-th stretch of
        // `stretch` positions (aligned to absolute position 0) that its queries can see
        const int s_abs = lo_first / stretch + blockIdx.z;
        if (s_abs * stretch > p_last) return;
        lo_first = max(lo_first, s_abs * stretch);
        p_last = min(p_last, (s_abs + 1) * stretch - 1);
    }
    const int* table = block_table + (size_t)r * max_blocks;
    rv_pdl_wait();

    // the block's query rows (zeros beyond its last token)
    for (int i = tid; i < AM_QT * (H * D / 2); i += blockDim.x) {
        const int row = i / (H * D / 2), c = i - row * (H * D / 2);
        ((unsigned*)(Qs + row * QS))[c] =
            row < n_q ? ((const unsigned*)(rows + (size_t)(q0 + t_first + row) * row_stride))[c] : 0u;
    }
    float o[2][DV / 8][4];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[hh][nt][i] = 0.f;

    // keys of tile j0 into Ks / values into Vs: a warp per key, 16-byte pieces, zeros where
    // nothing is seen
    const int nwarps = blockDim.x >> 5;
    auto load_tile = [&](int j0, bool keys) {
        const int chunks = (keys ? G * D : G * DV) / 8;
        bf16* dst = keys ? Ks : Vs;
        const bf16* src = keys ? k_cache : v_cache;
        const int stride = keys ? KS : VS;
        if (j0 <= p_last)
            for (int jj = warp; jj < AM_KT; jj += nwarps) {
                const int j = j0 + jj;
                bool valid = j >= lo_first && j <= p_last;
                long long slot = 0;
                if (valid) {
                    const int page = table[j / page_size];
                    valid = page >= 0;
                    slot = (long long)page * page_size + j % page_size;
                }
                for (int c = lane; c < chunks; c += 32)
                    am_cp_async_16(dst + jj * stride + c * 8, src + ((size_t)slot * chunks + c) * 8, valid);
            }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    const int j_first = lo_first / AM_KT * AM_KT;
    load_tile(j_first, true);
    load_tile(j_first, false);
    for (int j0 = j_first; j0 <= p_last; j0 += AM_KT) {
        // 1. the tile's keys have landed (its values may still be on their way)
        asm volatile("cp.async.wait_group 1;\n" ::);
        __syncthreads();
        // 2. raw scores of this warp's heads
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int h = 2 * warp + hh, g = h / hpg;
            float* Sh = S + (size_t)h * AM_QT * AM_SS;
            unsigned qf[D / 16][4];
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                am_ldmatrix_x4(qf[ks], Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * QS + h * D + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nt = 0; nt < AM_KT / 8; ++nt) {
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                const bf16* kb = Ks + (nt * 8 + (lane >> 2)) * KS + g * D + (lane & 3) * 2;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    am_mma(c, qf[ks], *(const unsigned*)(kb + ks * 16), *(const unsigned*)(kb + ks * 16 + 8));
                const int col = nt * 8 + (lane & 3) * 2;
                *(float2*)(Sh + (lane >> 2) * AM_SS + col) = make_float2(c[0] * scale2, c[1] * scale2);
                *(float2*)(Sh + ((lane >> 2) + 8) * AM_SS + col) = make_float2(c[2] * scale2, c[3] * scale2);
            }
        }
        __syncthreads();
        load_tile(j0 + AM_KT, true);          // the next tile's keys travel during the mixing
        // 3. mixing, mask, running softmax; token rows beyond the block's last token do nothing
        //    (the 8 lanes that share a token leave together, so the shuffles name only them)
        float acc[8][4];
        if (mq_live) {
            const unsigned gmask = 0xFFu << (lane & 24);
            // s'_h = sum_g M[h, g] s_g for 8 heads x 4 keys: packed float32 multiply-adds (two keys
            // an instruction), the coefficient in both halves
            unsigned long long acc2[8][2];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc2[j][0] = acc2[j][1] = 0ull;
            const float* sp = S + mq * AM_SS + kg * 4;
            const float* tp = Tt + hb * 16;
            for (int g = 0; g < H; ++g) {
                const ulonglong2 sv = *(const ulonglong2*)(sp + (size_t)g * AM_QT * AM_SS);
                const ulonglong2* tg = (const ulonglong2*)(tp + (size_t)g * H * 2);
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const ulonglong2 tv = tg[jj];
                    am_fma2(acc2[2 * jj][0], tv.x, sv.x);
                    am_fma2(acc2[2 * jj][1], tv.x, sv.y);
                    am_fma2(acc2[2 * jj + 1][0], tv.y, sv.x);
                    am_fma2(acc2[2 * jj + 1][1], tv.y, sv.y);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc[j][0] = __uint_as_float((unsigned)acc2[j][0]);
                acc[j][1] = __uint_as_float((unsigned)(acc2[j][0] >> 32));
                acc[j][2] = __uint_as_float((unsigned)acc2[j][1]);
                acc[j][3] = __uint_as_float((unsigned)(acc2[j][1] >> 32));
            }
            bool see[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int j = j0 + kg * 4 + i;
                see[i] = mq_live && j >= mlo && j <= mp;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float mx = -INFINITY;
#pragma unroll
                for (int i = 0; i < 4; ++i) mx = fmaxf(mx, see[i] ? acc[j][i] : -INFINITY);
                mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, 2));
                mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, 4));
                const int h = hb * 8 + j;
                const float m_old = m_s[h * AM_QT + mq], l_old = l_s[h * AM_QT + mq];
                __syncwarp(gmask);
                const float m_new = fmaxf(m_old, mx);
                float e[4];
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    e[i] = (see[i] && m_new != -INFINITY) ? exp2f(acc[j][i] - m_new) : 0.f;
                    e[i] = __bfloat162float(__float2bfloat16_rn(e[i]));
                    sum += e[i];
                }
                sum += __shfl_xor_sync(gmask, sum, 1);
                sum += __shfl_xor_sync(gmask, sum, 2);
                sum += __shfl_xor_sync(gmask, sum, 4);
                const float alpha = (m_old == -INFINITY) ? (m_new == -INFINITY ? 1.f : 0.f)
                                                         : exp2f(m_old - m_new);
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[j][i] = e[i];
                if (kg == 0) {
                    alpha_s[h * AM_QT + mq] = alpha;
                    m_s[h * AM_QT + mq] = m_new;
                    l_s[h * AM_QT + mq] = l_old * alpha + sum;
                }
            }
        }
        __syncthreads();
        // every score has been read: the probabilities take their place
        if (mq_live) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const __nv_bfloat162 p01 = __floats2bfloat162_rn(acc[j][0], acc[j][1]);
                const __nv_bfloat162 p23 = __floats2bfloat162_rn(acc[j][2], acc[j][3]);
                uint2 pk;
                pk.x = *(const unsigned*)&p01;
                pk.y = *(const unsigned*)&p23;
                *(uint2*)(P + ((size_t)(hb * 8 + j) * AM_QT + mq) * AM_PS + kg * 4) = pk;
            }
        }
        asm volatile("cp.async.wait_group 1;\n" ::);      // this tile's values have landed
        __syncthreads();
        // 4. O_h = alpha O_h + P_h V for this warp's heads
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int h = 2 * warp + hh, g = h / hpg;
            const float a_lo = alpha_s[h * AM_QT + (lane >> 2)], a_hi = alpha_s[h * AM_QT + (lane >> 2) + 8];
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt) {
                o[hh][nt][0] *= a_lo; o[hh][nt][1] *= a_lo;
                o[hh][nt][2] *= a_hi; o[hh][nt][3] *= a_hi;
            }
            const bf16* Ph = P + (size_t)h * AM_QT * AM_PS;
#pragma unroll
            for (int ks = 0; ks < AM_KT / 16; ++ks) {
                unsigned a[4];
                const bf16* pb = Ph + (lane >> 2) * AM_PS + ks * 16 + (lane & 3) * 2;
                a[0] = *(const unsigned*)pb;
                a[1] = *(const unsigned*)(pb + 8 * AM_PS);
                a[2] = *(const unsigned*)(pb + 8);
                a[3] = *(const unsigned*)(pb + 8 * AM_PS + 8);
#pragma unroll
                for (int nt = 0; nt < DV / 8; nt += 2) {
                    unsigned b[4];
                    // matrices: (keys 0..7, nt), (keys 8..15, nt), (keys 0..7, nt+1), (keys 8..15, nt+1)
                    const bf16* vb = Vs + (ks * 16 + (lane & 15)) * VS + g * DV + (nt + (lane >> 4)) * 8;
                    am_ldmatrix_x4_trans(b, vb);
                    am_mma(o[hh][nt], a, b[0], b[1]);
                    am_mma(o[hh][nt + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();
        load_tile(j0 + AM_KT, false);         // the next tile's values travel during its scores
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    const int n_out = H * DV;
    if (scratch) {
        // [token][stretch]: H maxima, H sums, H * DV unnormalised values; the merge kernel of
        // attention_mixed.cu puts a token's stretches together
        const size_t stride = (size_t)(2 * H + n_out);
        for (int i = tid; i < H * n_q; i += blockDim.x) {
            const int h = i / n_q, row = i - h * n_q;
            float* part = scratch + ((size_t)(q0 + t_first + row - first_token) * gridDim.z + blockIdx.z) * stride;
            part[h] = m_s[h * AM_QT + row] * AM_LN2;           // the merge works with natural logarithms
            part[H + h] = l_s[h * AM_QT + row];
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int h = 2 * warp + hh;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = (lane >> 2) + 8 * half;
                if (row >= n_q) continue;
                float* part = scratch + ((size_t)(q0 + t_first + row - first_token) * gridDim.z + blockIdx.z) * stride + 2 * H;
#pragma unroll
                for (int nt = 0; nt < DV / 8; ++nt)
                    *(float2*)(part + h * DV + nt * 8 + (lane & 3) * 2) =
                        make_float2(o[hh][nt][2 * half], o[hh][nt][2 * half + 1]);
            }
        }
        return;
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int h = 2 * warp + hh;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = (lane >> 2) + 8 * half;
            if (row >= n_q) continue;
            const float l = l_s[h * AM_QT + row];
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const size_t t = (size_t)(q0 + t_first + row);
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt) {
                const int e = h * DV + nt * 8 + (lane & 3) * 2;
                float y0 = o[hh][nt][2 * half] * inv, y1 = o[hh][nt][2 * half + 1] * inv;
                if (gate_off >= 0) {
                    const float2 gt = __bfloat1622float2(*(const __nv_bfloat162*)(rows + t * row_stride + gate_off + e));
                    y0 *= 1.f / (1.f + expf(-gt.x));
                    y1 *= 1.f / (1.f + expf(-gt.y));
                }
                *(__nv_bfloat162*)(out + t * n_out + e) = __floats2bfloat162_rn(y0, y1);
            }
        }
    }
}

extern "C" long long AM_NAME(rv_attention_mixed_mma_smem_d)(int H, int G) {
    return (long long)AM_KT * (G * RV_D + 8) * 2 + (long long)AM_KT * (G * RV_DV + 8) * 2 +
           (long long)H * AM_QT * AM_SS * 4 + (long long)AM_QT * (H * RV_D + 8) * 2 + (long long)H * H * 8 +
           3ll * H * AM_QT * 4;
}

// Requests [first_req, first_req + n_reqs) bring `max_q_len` tokens at most.
extern "C" int AM_NAME(rv_attention_mixed_mma_d)(
    const void* rows, int row_stride, int gate_off, const void* k_cache, const void* v_cache,
    const int* block_table, int max_blocks, const int* q_start, const int* ctx_lens, void* out,
    int first_req, int n_reqs, int max_q_len, int H, int G, int page_size, float scale, int window,
    int chunk, const float* mix, const float* sinks, float* scratch, int stretch, int n_stretch,
    int first_token, void* stream) {
    // `scratch` given: every block's keys are shared out over up to `n_stretch` blocks, one per
    // `stretch` positions, which leave partial results there for the merge kernel; it holds
    // (tokens from `first_token` on) * n_stretch * (2 H + H dv) floats
    if (n_reqs <= 0 || max_q_len <= 0) return 0;
    if (H <= 0 || H % 8 || H > 32 || G <= 0 || H % G) AM_FAIL("attention_mixed_mma: %d heads (multiples of 8 up to 32) over %d key/value heads", H, G);
    if (row_stride % 2 || (gate_off >= 0 && gate_off % 2) || ((uintptr_t)rows % 4) || ((uintptr_t)out % 4) ||
        ((uintptr_t)k_cache % 16) || ((uintptr_t)v_cache % 16))
        AM_FAIL("attention_mixed_mma: rows or pages are not aligned");
    const long long smem = AM_NAME(rv_attention_mixed_mma_smem_d)(H, G);
    if (smem > 227 * 1024) AM_FAIL("attention_mixed_mma: %lld bytes of shared memory", smem);
    auto kernel = H <= 16 ? attention_mixed_mma_kernel<256> : attention_mixed_mma_kernel<512>;
    static long long configured[2] = {0, 0};
    if (smem > configured[H > 16]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) AM_FAIL("attention_mixed_mma: %s", cudaGetErrorString(e));
        configured[H > 16] = smem;
    }
    if (scratch && (stretch <= 0 || stretch % AM_KT || n_stretch <= 0)) AM_FAIL("attention_mixed_mma: bad stretch");
    rv_launch(kernel, dim3((max_q_len + AM_QT - 1) / AM_QT, n_reqs, scratch ? n_stretch : 1), dim3(16 * H),
              (size_t)smem, (cudaStream_t)stream, (const bf16*)rows, row_stride, gate_off,
              (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_blocks, q_start, ctx_lens,
              (bf16*)out, first_req, H, G, page_size, scale, window, chunk, mix, sinks, scratch,
              stretch, first_token);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) AM_FAIL("attention_mixed_mma: %s", cudaGetErrorString(e));
    return 0;
}
