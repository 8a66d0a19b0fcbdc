// Paged attention whose heads are mixed before the softmax, float32 arithmetic for any storage
// type: every head of a query token is computed by one block, because no head's softmax can
// be formed without the other heads' scores.
//
// rows [N, row_stride]: q of H heads of size d at the front; at `gate_off` (>= 0) H*dv gate
// values.  For the token at position p, over the visible keys j in [lo, p],
// lo = max(0, p - window + 1 (window > 0), floor(p / chunk) * chunk (chunk > 0)):
//     s_g[j]  = scale * <q_g, k_kv(g)[j]>
//     s'_h[j] = sum_g mix[h, g] s_g[j]                       (mix given; else s' = s)
//     w_h[j]  = exp(s'_h[j]) / (sum_j' exp(s'_h[j']) + exp(sink_h))   (sinks given)
//     out_h   = sum_j w_h[j] v_kv(h)[j]   * sigmoid(gate_h)          (gate_off >= 0)
// Keys are walked in tiles of 32 aligned to absolute position 0, with a running maximum and
// sum per head, so a position's result does not depend on how its prompt was cut.  The sink
// enters as the initial maximum and a sum of 1.
// Plain reference: tests/plain_ops.py paged_attention_mixed.
#include "common.cuh"

#define AM_KT 32          // keys per tile
#define AM_THREADS 256
#define AM_MAX_ACC 16     // H * dv <= AM_THREADS * AM_MAX_ACC
#define AM_MAX_KREG 8     // d <= 32 * AM_MAX_KREG

template <typename T>
__global__ void paged_attention_mixed_kernel(
    const T* __restrict__ rows, int row_stride, int gate_off, const T* __restrict__ k_cache,
    const T* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ q_start, const int* __restrict__ ctx_lens,
    const int* __restrict__ token_req, T* __restrict__ out, int first_token, int H, int G, int d,
    int dv, int page_size, float scale, int window, int chunk, const float* __restrict__ mix,
    const float* __restrict__ sinks) {
    rv_pdl_launch_dependents();
    extern __shared__ float smem[];
    float* q_s = smem;                       // [H * d]
    float* mix_s = q_s + H * d;              // [H * H]
    float* raw_s = mix_s + H * H;            // [H * KT]
    float* p_s = raw_s + H * AM_KT;          // [H * KT]
    float* m_s = p_s + H * AM_KT;            // [H]
    float* l_s = m_s + H;                    // [H]
    float* alpha_s = l_s + H;                // [H]
    long long* slot_s = (long long*)(((uintptr_t)(alpha_s + H) + 7) & ~(uintptr_t)7);   // [KT]
    const int t = first_token + blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int r = token_req[t];
    const int clen = ctx_lens[r];
    if (clen == 0) return;                                     // a padding request
    const int p = clen - (q_start[r + 1] - q_start[r]) + (t - q_start[r]);
    int lo = 0;
    if (window > 0) lo = max(lo, p - window + 1);
    if (chunk > 0) lo = max(lo, p / chunk * chunk);
    if (mix)
        for (int i = tid; i < H * H; i += blockDim.x) mix_s[i] = mix[i];
    for (int h = tid; h < H; h += blockDim.x) {
        m_s[h] = sinks ? sinks[h] : -INFINITY;
        l_s[h] = sinks ? 1.f : 0.f;
    }
    rv_pdl_wait();
    const T* row = rows + (size_t)t * row_stride;
    for (int i = tid; i < H * d; i += blockDim.x) q_s[i] = rv_load(row + i);
    const int hpg = H / G;
    const int n_out = H * dv;
    float acc[AM_MAX_ACC];
#pragma unroll
    for (int i = 0; i < AM_MAX_ACC; ++i) acc[i] = 0.f;
    const int* table = block_table + (size_t)r * max_blocks;
    __syncthreads();
    for (int j0 = lo / AM_KT * AM_KT; j0 <= p; j0 += AM_KT) {
        if (tid < AM_KT) {
            const int j = j0 + tid;
            long long s = -1;
            if (j >= lo && j <= p) {
                const int page = table[j / page_size];
                if (page >= 0) s = (long long)page * page_size + j % page_size;
            }
            slot_s[tid] = s;
        }
        __syncthreads();
        // raw scores: a warp takes (kv head, key) pairs, holds the key in registers and serves
        // the query heads of its group
        for (int pair = warp; pair < G * AM_KT; pair += nwarps) {
            const int g = pair / AM_KT, jj = pair - g * AM_KT;
            const long long s = slot_s[jj];
            if (s < 0) {
                if (lane < hpg) raw_s[(g * hpg + lane) * AM_KT + jj] = 0.f;
                for (int hh = 32 + lane; hh < hpg; hh += 32) raw_s[(g * hpg + hh) * AM_KT + jj] = 0.f;
                continue;
            }
            const T* kp = k_cache + ((size_t)s * G + g) * d;
            float kr[AM_MAX_KREG];
#pragma unroll
            for (int i = 0; i < AM_MAX_KREG; ++i) kr[i] = (lane + 32 * i < d) ? rv_load(kp + lane + 32 * i) : 0.f;
            for (int hh = 0; hh < hpg; ++hh) {
                const float* qh = q_s + (size_t)(g * hpg + hh) * d;
                float dot = 0.f;
#pragma unroll
                for (int i = 0; i < AM_MAX_KREG; ++i)
                    if (lane + 32 * i < d) dot += qh[lane + 32 * i] * kr[i];
                dot = rv_warp_sum(dot);
                if (lane == 0) raw_s[(g * hpg + hh) * AM_KT + jj] = dot * scale;
            }
        }
        __syncthreads();
        // mixing over the heads, and the mask
        for (int i = tid; i < H * AM_KT; i += blockDim.x) {
            const int h = i / AM_KT, jj = i - h * AM_KT;
            float v = -INFINITY;
            if (slot_s[jj] >= 0) {
                if (mix) {
                    v = 0.f;
                    for (int g = 0; g < H; ++g) v += mix_s[h * H + g] * raw_s[g * AM_KT + jj];
                } else {
                    v = raw_s[i];
                }
            }
            p_s[i] = v;
        }
        __syncthreads();
        // running maximum and sum per head: a warp per head, a lane per key of the tile
        for (int h = warp; h < H; h += nwarps) {
            const float v = p_s[h * AM_KT + lane];
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, rv_warp_max(v));
            const float e = (v == -INFINITY) ? 0.f : expf(v - m_new);
            const float sum = rv_warp_sum(e);
            const float alpha = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
            p_s[h * AM_KT + lane] = e;
            if (lane == 0) {
                m_s[h] = m_new;
                l_s[h] = l_s[h] * alpha + sum;
                alpha_s[h] = alpha;
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < AM_MAX_ACC; ++i) {
            const int e = tid + i * AM_THREADS;
            if (e < n_out) {
                const int h = e / dv, dd = e - h * dv, g = h / hpg;
                float a = acc[i] * alpha_s[h];
                const float* ph = p_s + h * AM_KT;
                for (int jj = 0; jj < AM_KT; ++jj) {
                    const long long s = slot_s[jj];
                    if (s >= 0) a += ph[jj] * rv_load(v_cache + ((size_t)s * G + g) * dv + dd);
                }
                acc[i] = a;
            }
        }
        __syncthreads();
    }
    T* o = out + (size_t)t * n_out;
#pragma unroll
    for (int i = 0; i < AM_MAX_ACC; ++i) {
        const int e = tid + i * AM_THREADS;
        if (e < n_out) {
            const int h = e / dv;
            const float l = l_s[h];
            float y = l > 0.f ? acc[i] / l : 0.f;
            if (gate_off >= 0) y *= 1.f / (1.f + expf(-rv_load(row + gate_off + e)));
            rv_store(o + e, y);
        }
    }
}

extern "C" int rv_paged_attention_mixed(
    const void* rows, int dtype, int row_stride, int gate_off, const void* k_cache,
    const void* v_cache, const int* block_table, int max_blocks, const int* q_start,
    const int* ctx_lens, const int* token_req, void* out, int first_token, int n_tokens, int H,
    int G, int d, int dv, int page_size, float scale, int window, int chunk, const float* mix,
    const float* sinks, void* stream) {
    if (n_tokens == 0) return 0;
    if (n_tokens < 0 || H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || page_size <= 0)
        RV_FAIL("paged_attention_mixed: bad sizes");
    if (d > 32 * AM_MAX_KREG) RV_FAIL("paged_attention_mixed: head size %d exceeds %d", d, 32 * AM_MAX_KREG);
    if (H * dv > AM_THREADS * AM_MAX_ACC)
        RV_FAIL("paged_attention_mixed: %d heads of %d values exceed %d outputs a token", H, dv,
                AM_THREADS * AM_MAX_ACC);
    const size_t smem = sizeof(float) * ((size_t)H * d + (size_t)H * H + 2 * (size_t)H * AM_KT + 3 * H + 1) +
                        sizeof(long long) * AM_KT + 8;
    if (smem > 200 * 1024) RV_FAIL("paged_attention_mixed: %d heads of size %d do not fit shared memory", H, d);
    cudaStream_t s = (cudaStream_t)stream;
    RV_DISPATCH_DTYPE(dtype, "paged_attention_mixed", {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(paged_attention_mixed_kernel<T>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) RV_FAIL("paged_attention_mixed: %s", cudaGetErrorString(e));
        }
        rv_launch(paged_attention_mixed_kernel<T>, dim3(n_tokens), dim3(AM_THREADS), smem, s,
                  (const T*)rows, row_stride, gate_off, (const T*)k_cache, (const T*)v_cache,
                  block_table, max_blocks, q_start, ctx_lens, token_req, (T*)out, first_token, H, G,
                  d, dv, page_size, scale, window, chunk, mix, sinks);
    });
    RV_CHECK_LAUNCH("paged_attention_mixed");
    return 0;
}
