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
// Single tokens (decoding) are split over the keys: block (token, s) takes the keys of the
// s-th stretch of AM_SPLIT positions (aligned to absolute position 0) that the token sees and
// leaves its running maximum, sum and unnormalised values in a scratch buffer; a second kernel
// puts a token's stretches together in order, adds the sink once, divides and gates.  Which
// stretches a token has depends on its own position only.
// Plain reference: tests/plain_ops.py paged_attention_mixed.
#include "common.cuh"

#define AM_SPLIT 128      // keys per block of a split launch (a multiple of AM_KT)

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
    const int hi = p;                                          // the block's keys: [lo, hi]
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
    for (int j0 = lo / AM_KT * AM_KT; j0 <= hi; j0 += AM_KT) {
        if (tid < AM_KT) {
            const int j = j0 + tid;
            long long s = -1;
            if (j >= lo && j <= hi) {
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

// Single tokens, split over the keys.  Block (token, s) stages tiles of 32 keys and values of
// its stretch in shared memory (rows padded to an odd number of 32-bit words, so that a warp
// whose lanes walk 32 keys meets no bank twice).  Raw scores: a warp per key/value head, a lane
// per key, the key's values read once for up to four query heads of the group.  Mixing: a thread
// per (four heads, key) with the mixing matrix transposed, so that one score meets four
// coefficients in one 16-byte load.  Running maximum and sum: a warp per head.  Values: a thread
// per (four heads, two neighbouring value dimensions), probabilities transposed to [key][head].
#define AM_SPLIT_ITEMS 2      // (four heads x two dimensions) items a thread: H * dv <= 4096

template <typename T>
__global__ void paged_attention_mixed_split_kernel(
    const T* __restrict__ rows, int row_stride, const T* __restrict__ k_cache,
    const T* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ q_start, const int* __restrict__ ctx_lens,
    const int* __restrict__ token_req, int first_token, int H, int G, int d, int dv, int page_size,
    float scale, int window, int chunk, const float* __restrict__ mix,
    float* __restrict__ scratch, int n_splits) {
    rv_pdl_launch_dependents();
    constexpr int PER = 4 / sizeof(T);                 // elements per 32-bit word
    const int kw = G * d / PER + 1, vw = G * dv / PER + 1;          // row lengths in words (odd)
    const int HP = (H + 3) & ~3, HPP = HP + 4;
    extern __shared__ __align__(16) float smem[];
    float* mixT = smem;                                // [H][HP]: mixT[g][h] = mix[h][g]
    float* p_t = mixT + H * HP;                        // [KT][HPP] probabilities, transposed
    float* q_s = p_t + AM_KT * HPP;                    // [H * d]
    float* raw_s = q_s + ((H * d + 3) & ~3);           // [H][KT + 1]
    float* p_s = raw_s + H * (AM_KT + 1);              // [H][KT + 1] mixed scores
    float* m_s = p_s + H * (AM_KT + 1);                // [H]
    float* l_s = m_s + H;
    float* alpha_s = l_s + H;                          // [HP]
    unsigned* kt = (unsigned*)(alpha_s + HP);          // [KT][kw] words
    unsigned* vt = kt + AM_KT * kw;                    // [KT][vw] words
    __shared__ long long slot_s[AM_KT];
    const int t = first_token + blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int r = token_req[t];
    const int clen = ctx_lens[r];
    if (clen == 0) return;                                     // a padding request
    const int p = clen - (q_start[r + 1] - q_start[r]) + (t - q_start[r]);
    int lo = 0;
    if (window > 0) lo = max(lo, p - window + 1);
    if (chunk > 0) lo = max(lo, p / chunk * chunk);
    const int s_abs = lo / AM_SPLIT + blockIdx.y;
    if (s_abs * AM_SPLIT > p) return;                          // the token has fewer stretches
    lo = max(lo, s_abs * AM_SPLIT);
    const int hi = min(p, (s_abs + 1) * AM_SPLIT - 1);
    for (int i = tid; i < H * HP; i += blockDim.x) {
        const int g = i / HP, h = i - g * HP;
        mixT[i] = h < H ? (mix ? mix[h * H + g] : (g == h ? 1.f : 0.f)) : 0.f;
    }
    for (int h = tid; h < HP; h += blockDim.x) {
        if (h < H) {
            m_s[h] = -INFINITY;
            l_s[h] = 0.f;
        }
        alpha_s[h] = 0.f;
    }
    for (int i = tid; i < AM_KT * HPP; i += blockDim.x) p_t[i] = 0.f;
    rv_pdl_wait();
    const T* row = rows + (size_t)t * row_stride;
    for (int i = tid; i < H * d; i += blockDim.x) q_s[i] = rv_load(row + i);
    const int hpg = H / G;
    const int n_out = H * dv;
    const bool one_group = hpg % 4 == 0;                       // four neighbouring heads share their values
    const int n_items = (HP / 4) * (dv / 2);
    float acc[AM_SPLIT_ITEMS][8];
#pragma unroll
    for (int i = 0; i < AM_SPLIT_ITEMS; ++i)
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[i][u] = 0.f;
    const int* table = block_table + (size_t)r * max_blocks;
    const int krow = G * d / PER, vrow = G * dv / PER;         // words of a key / value row
    const bool vec16 = krow % 4 == 0 && vrow % 4 == 0 && (uintptr_t)k_cache % 16 == 0 &&
                       (uintptr_t)v_cache % 16 == 0;
    for (int j0 = lo / AM_KT * AM_KT; j0 <= hi; j0 += AM_KT) {
        __syncthreads();                                       // the previous tile is used up
        if (tid < AM_KT) {
            const int j = j0 + tid;
            long long s = -1;
            if (j >= lo && j <= hi) {
                const int page = table[j / page_size];
                if (page >= 0) s = (long long)page * page_size + j % page_size;
            }
            slot_s[tid] = s;
        }
        __syncthreads();
        if (vec16) {
            // a warp per key: 16-byte loads, up to four in flight per lane before any is stored
            const int kq = krow / 4, per = kq + vrow / 4;
            for (int jj = warp; jj < AM_KT; jj += nwarps) {
                const long long s = slot_s[jj];
                const uint4* ksrc = (const uint4*)k_cache + (size_t)(s < 0 ? 0 : s) * kq;
                const uint4* vsrc = (const uint4*)v_cache + (size_t)(s < 0 ? 0 : s) * (per - kq);
                for (int c0 = lane; c0 < per; c0 += 128) {
                    uint4 val[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int c = c0 + 32 * u;
                        val[u] = make_uint4(0u, 0u, 0u, 0u);
                        if (c < per && s >= 0) val[u] = c < kq ? ksrc[c] : vsrc[c - kq];
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int c = c0 + 32 * u;
                        if (c < per) {
                            unsigned* dst = c < kq ? kt + jj * kw + 4 * c : vt + jj * vw + 4 * (c - kq);
                            dst[0] = val[u].x; dst[1] = val[u].y; dst[2] = val[u].z; dst[3] = val[u].w;
                        }
                    }
                }
            }
        } else {
            for (int jj = warp; jj < AM_KT; jj += nwarps) {
                const long long s = slot_s[jj];
                for (int c = lane; c < krow; c += 32)
                    kt[jj * kw + c] = s < 0 ? 0u : ((const unsigned*)k_cache)[(size_t)s * krow + c];
                for (int c = lane; c < vrow; c += 32)
                    vt[jj * vw + c] = s < 0 ? 0u : ((const unsigned*)v_cache)[(size_t)s * vrow + c];
            }
        }
        __syncthreads();
        // raw scores: a warp per key/value head, a lane per key, four query heads at a time
        for (int g = warp; g < G; g += nwarps) {
            const T* kr = (const T*)(kt + lane * kw) + g * d;
            for (int hh0 = 0; hh0 < hpg; hh0 += 4) {
                float dot[4] = {0.f, 0.f, 0.f, 0.f};
                const int nh = min(4, hpg - hh0);
                const float* qh = q_s + (size_t)(g * hpg + hh0) * d;
                // heads beyond the group read the group's last head again; their sums are dropped
                const float* q0 = qh, *q1 = qh + min(1, nh - 1) * d, *q2 = qh + min(2, nh - 1) * d,
                           *q3 = qh + min(3, nh - 1) * d;
#pragma unroll 4
                for (int i = 0; i < d; i += 2) {
                    float k0, k1;
                    if (sizeof(T) == 2) {
                        const float2 kk = __bfloat1622float2(*(const __nv_bfloat162*)(kr + i));
                        k0 = kk.x;
                        k1 = kk.y;
                    } else {
                        k0 = rv_load(kr + i);
                        k1 = rv_load(kr + i + 1);
                    }
                    const float2 a0 = *(const float2*)(q0 + i), a1 = *(const float2*)(q1 + i),
                                 a2 = *(const float2*)(q2 + i), a3 = *(const float2*)(q3 + i);
                    dot[0] += a0.x * k0 + a0.y * k1;
                    dot[1] += a1.x * k0 + a1.y * k1;
                    dot[2] += a2.x * k0 + a2.y * k1;
                    dot[3] += a3.x * k0 + a3.y * k1;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (u < nh) raw_s[(g * hpg + hh0 + u) * (AM_KT + 1) + lane] = dot[u] * scale;
            }
        }
        __syncthreads();
        // mixing over the heads, and the mask: a thread per (four heads, key)
        for (int i = tid; i < (HP / 4) * AM_KT; i += blockDim.x) {
            const int hq = i / AM_KT, jj = i - hq * AM_KT;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            const bool seen = slot_s[jj] >= 0;
            if (seen)
#pragma unroll 8
                for (int g = 0; g < H; ++g) {
                    const float rw = raw_s[g * (AM_KT + 1) + jj];
                    const float4 m4 = *(const float4*)(mixT + g * HP + hq * 4);
                    v[0] += m4.x * rw; v[1] += m4.y * rw; v[2] += m4.z * rw; v[3] += m4.w * rw;
                }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (hq * 4 + u < H) p_s[(hq * 4 + u) * (AM_KT + 1) + jj] = seen ? v[u] : -INFINITY;
        }
        __syncthreads();
        for (int h = warp; h < H; h += nwarps) {
            const float v = p_s[h * (AM_KT + 1) + lane];
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, rv_warp_max(v));
            const float e = (v == -INFINITY) ? 0.f : expf(v - m_new);
            const float sum = rv_warp_sum(e);
            const float alpha = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
            p_t[lane * HPP + h] = e;
            if (lane == 0) {
                m_s[h] = m_new;
                l_s[h] = l_s[h] * alpha + sum;
                alpha_s[h] = alpha;
            }
        }
        __syncthreads();
        // values: a thread per (four heads, two neighbouring dimensions)
#pragma unroll
        for (int it = 0; it < AM_SPLIT_ITEMS; ++it) {
            const int item = tid + it * AM_THREADS;
            if (item < n_items) {
                const int hq = item / (dv / 2), dd = (item - hq * (dv / 2)) * 2;
                const float4 al = *(const float4*)(alpha_s + hq * 4);
                acc[it][0] *= al.x; acc[it][1] *= al.x; acc[it][2] *= al.y; acc[it][3] *= al.y;
                acc[it][4] *= al.z; acc[it][5] *= al.z; acc[it][6] *= al.w; acc[it][7] *= al.w;
                if (one_group) {
                    const T* vcol = (const T*)vt + (hq * 4 / hpg) * dv + dd;
#pragma unroll 8
                    for (int jj = 0; jj < AM_KT; ++jj) {
                        const float4 pr = *(const float4*)(p_t + jj * HPP + hq * 4);
                        const T* vp = vcol + (size_t)jj * vw * PER;
                        float v0, v1;
                        if (sizeof(T) == 2) {
                            const float2 vv = __bfloat1622float2(*(const __nv_bfloat162*)vp);
                            v0 = vv.x;
                            v1 = vv.y;
                        } else {
                            v0 = rv_load(vp);
                            v1 = rv_load(vp + 1);
                        }
                        acc[it][0] += pr.x * v0; acc[it][1] += pr.x * v1;
                        acc[it][2] += pr.y * v0; acc[it][3] += pr.y * v1;
                        acc[it][4] += pr.z * v0; acc[it][5] += pr.z * v1;
                        acc[it][6] += pr.w * v0; acc[it][7] += pr.w * v1;
                    }
                } else {
                    for (int jj = 0; jj < AM_KT; ++jj) {
                        const float4 pr = *(const float4*)(p_t + jj * HPP + hq * 4);
                        const float pu[4] = {pr.x, pr.y, pr.z, pr.w};
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int h = min(hq * 4 + u, H - 1);
                            const T* vp = (const T*)vt + (size_t)jj * vw * PER + (h / hpg) * dv + dd;
                            acc[it][2 * u] += pu[u] * rv_load(vp);
                            acc[it][2 * u + 1] += pu[u] * rv_load(vp + 1);
                        }
                    }
                }
            }
        }
    }
    // [token][stretch]: H maxima, H sums, H * dv unnormalised values
    float* part = scratch + ((size_t)blockIdx.x * n_splits + blockIdx.y) * (size_t)(2 * H + n_out);
    __syncthreads();
    for (int h = tid; h < H; h += blockDim.x) {
        part[h] = m_s[h];
        part[H + h] = l_s[h];
    }
#pragma unroll
    for (int it = 0; it < AM_SPLIT_ITEMS; ++it) {
        const int item = tid + it * AM_THREADS;
        if (item < n_items) {
            const int hq = item / (dv / 2), dd = (item - hq * (dv / 2)) * 2;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (hq * 4 + u < H) {
                    part[2 * H + (hq * 4 + u) * dv + dd] = acc[it][2 * u];
                    part[2 * H + (hq * 4 + u) * dv + dd + 1] = acc[it][2 * u + 1];
                }
        }
    }
}

// One block per single token: its stretches in order, the sink once, the division, the gate.
template <typename T>
__global__ void paged_attention_mixed_merge_kernel(
    const float* __restrict__ scratch, int n_splits, const T* __restrict__ rows, int row_stride,
    int gate_off, const int* __restrict__ q_start, const int* __restrict__ ctx_lens,
    const int* __restrict__ token_req, T* __restrict__ out, int first_token, int H, int dv,
    int window, int chunk, const float* __restrict__ sinks, int stretch, int tile) {
    // `tile`: how many neighbouring tokens of a request shared one block of the split launch
    // (1: single tokens; 16: the tensor-core kernel's query tiles, counted from the request's
    // first token of the step); the stretches that ran are those the whole tile can see
    rv_pdl_prologue();
    const int t = first_token + blockIdx.x;
    const int r = token_req[t];
    const int clen = ctx_lens[r];
    if (clen == 0) return;
    const int q_len = q_start[r + 1] - q_start[r];
    const int in_tile = (t - q_start[r]) % tile;
    const int p_first = clen - q_len + (t - q_start[r]) - in_tile;
    const int p = min(p_first + tile - 1, clen - 1);           // the tile's last position
    int lo = 0;
    if (window > 0) lo = max(lo, p_first - window + 1);
    if (chunk > 0) lo = max(lo, p_first / chunk * chunk);
    const int n = p / stretch - lo / stretch + 1;              // stretches that ran
    const int n_out = H * dv;
    const size_t stride = (size_t)(2 * H + n_out);
    const float* base = scratch + (size_t)blockIdx.x * n_splits * stride;
    for (int e = threadIdx.x; e < n_out; e += blockDim.x) {
        const int h = e / dv;
        float m = sinks ? sinks[h] : -INFINITY;
        for (int s = 0; s < n; ++s) m = fmaxf(m, base[s * stride + h]);
        float l = sinks ? expf(sinks[h] - m) : 0.f;
        float a = 0.f;
        for (int s = 0; s < n; ++s) {
            const float ms = base[s * stride + h];
            const float w = (ms == -INFINITY) ? 0.f : expf(ms - m);
            l += base[s * stride + H + h] * w;
            a += base[s * stride + 2 * H + e] * w;
        }
        float y = l > 0.f ? a / l : 0.f;
        if (gate_off >= 0) y *= 1.f / (1.f + expf(-rv_load(rows + (size_t)t * row_stride + gate_off + e)));
        rv_store(out + (size_t)t * n_out + e, y);
    }
}

// Stretches a single token can have when it sees at most `span` keys.
extern "C" int rv_paged_attention_mixed_splits(int span) {
    return (span < 1 ? 1 : span + AM_SPLIT - 1) / AM_SPLIT + 1;
}
extern "C" long long rv_paged_attention_mixed_scratch_bytes(int n_tokens, int H, int dv, int span) {
    return (long long)n_tokens * rv_paged_attention_mixed_splits(span) * (2ll * H + (long long)H * dv) * 4;
}

// The merge alone, for partial results that the tensor-core kernel left: tokens
// [first_token, first_token + n_tokens), `n_splits` stretches of `stretch` positions each at
// most, tiles of `tile` query tokens.
extern "C" int rv_paged_attention_mixed_merge(
    const float* scratch, int n_splits, const void* rows, int dtype, int row_stride, int gate_off,
    const int* q_start, const int* ctx_lens, const int* token_req, void* out, int first_token,
    int n_tokens, int H, int dv, int window, int chunk, const float* sinks, int stretch, int tile,
    void* stream) {
    if (n_tokens <= 0) return 0;
    if (!scratch || n_splits <= 0 || stretch <= 0 || tile <= 0) RV_FAIL("paged_attention_mixed_merge: bad sizes");
    RV_DISPATCH_DTYPE(dtype, "paged_attention_mixed_merge",
                      (rv_launch(paged_attention_mixed_merge_kernel<T>, dim3(n_tokens), dim3(256), 0,
                                 (cudaStream_t)stream, scratch, n_splits, (const T*)rows, row_stride,
                                 gate_off, q_start, ctx_lens, token_req, (T*)out, first_token, H, dv,
                                 window, chunk, sinks, stretch, tile)));
    RV_CHECK_LAUNCH("paged_attention_mixed_merge");
    return 0;
}

extern "C" int rv_paged_attention_mixed(
    const void* rows, int dtype, int row_stride, int gate_off, const void* k_cache,
    const void* v_cache, const int* block_table, int max_blocks, const int* q_start,
    const int* ctx_lens, const int* token_req, void* out, int first_token, int n_tokens, int H,
    int G, int d, int dv, int page_size, float scale, int window, int chunk, const float* mix,
    const float* sinks, float* scratch, long long scratch_bytes, int span, void* stream) {
    // `scratch` given: the tokens are single tokens that see at most `span` keys each, and every
    // one is split over its keys
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
    if (scratch) {
        const int n_splits = rv_paged_attention_mixed_splits(span);
        if (rv_paged_attention_mixed_scratch_bytes(n_tokens, H, dv, span) > scratch_bytes)
            RV_FAIL("paged_attention_mixed: the scratch buffer is too small");
        const int el = dtype == RV_DTYPE_BF16 ? 2 : 4;
        if ((G * d * el) % 8 || (G * dv * el) % 8 || (uintptr_t)k_cache % 4 || (uintptr_t)v_cache % 4 || d % 2 || dv % 2)
            RV_FAIL("paged_attention_mixed: key and value rows of %d and %d bytes cannot be staged", G * d * el, G * dv * el);
        const int HP = (H + 3) & ~3;
        if ((HP / 4) * (dv / 2) > AM_SPLIT_ITEMS * AM_THREADS)
            RV_FAIL("paged_attention_mixed: %d heads of %d values exceed the split kernel", H, dv);
        const size_t ssmem = sizeof(float) * ((size_t)H * HP + (size_t)AM_KT * (HP + 4) + (((size_t)H * d + 3) & ~(size_t)3) +
                                              2 * (size_t)H * (AM_KT + 1) + 2 * H + HP) +
                             4 * (size_t)AM_KT * ((size_t)G * d * el / 4 + 1 + (size_t)G * dv * el / 4 + 1);
        if (ssmem > 200 * 1024) RV_FAIL("paged_attention_mixed: %d heads of size %d do not fit shared memory", H, d);
        RV_DISPATCH_DTYPE(dtype, "paged_attention_mixed", {
            if (ssmem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(paged_attention_mixed_split_kernel<T>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ssmem);
                if (e != cudaSuccess) RV_FAIL("paged_attention_mixed: %s", cudaGetErrorString(e));
            }
            rv_launch(paged_attention_mixed_split_kernel<T>, dim3(n_tokens, n_splits), dim3(AM_THREADS),
                      ssmem, s, (const T*)rows, row_stride, (const T*)k_cache, (const T*)v_cache,
                      block_table, max_blocks, q_start, ctx_lens, token_req, first_token, H, G, d, dv,
                      page_size, scale, window, chunk, mix, scratch, n_splits);
            rv_launch(paged_attention_mixed_merge_kernel<T>, dim3(n_tokens), dim3(256), 0, s,
                      (const float*)scratch, n_splits, (const T*)rows, row_stride, gate_off, q_start,
                      ctx_lens, token_req, (T*)out, first_token, H, dv, window, chunk, sinks, AM_SPLIT, 1);
        });
        RV_CHECK_LAUNCH("paged_attention_mixed");
        return 0;
    }
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
