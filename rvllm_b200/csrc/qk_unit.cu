// Finishing of a fused q|k|v product's rows for an attention without rotation, and the write
// of keys and values into the paged cache.  Rows are laid out as
//   [ q: H heads of d | k: G heads of d | v: G heads of dv | anything else ]
// (G = 0: the rows carry queries only and no cache is written).
//   unit norm (norm != 0): every q and k head is divided by sqrt(mean(x^2) + eps); no weight.
//   query temperature (every > 0): the query at position p is multiplied by
//       1 + coef * ln(floor((p + 1) / every) + 1).
// Queries are finished in place, keys go to the key pages, values as they are to the value
// pages.  Sums, the root, the logarithm and the products are float32; a result is rounded
// once, to the storage type.  One warp per (token, head).
// Plain reference: tests/plain_ops.py qk_unit_write.
#include "common.cuh"

template <typename T>
__global__ void qk_unit_write_kernel(T* __restrict__ rows, int row_stride, int n_tokens, int H,
                                     int G, int d, int dv, int norm, float eps, float coef,
                                     int every, const int* __restrict__ positions,
                                     const int* __restrict__ slot_mapping, T* __restrict__ k_cache,
                                     T* __restrict__ v_cache) {
    rv_pdl_launch_dependents();
    const int heads_total = H + 2 * G;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= (long long)n_tokens * heads_total) return;
    const int t = (int)(warp / heads_total);
    const int h = (int)(warp - (long long)t * heads_total);
    const int slot = h >= H ? slot_mapping[t] : 0;
    float temp = 1.f;
    if (h < H && every > 0)
        temp = 1.f + coef * logf((float)((positions[t] + 1) / every + 1));
    rv_pdl_wait();
    if (h >= H && slot < 0) return;
    T* row = rows + (size_t)t * row_stride;
    if (h >= H + G) {                                          // a value head: copy
        const int g = h - H - G;
        const T* src = row + (size_t)(H + G) * d + (size_t)g * dv;
        T* dst = v_cache + ((size_t)slot * G + g) * dv;
        for (int i = lane; i < dv; i += 32) dst[i] = src[i];
        return;
    }
    T* src = row + (size_t)h * d;                              // q heads, then k heads
    T* dst = h < H ? src : k_cache + ((size_t)slot * G + (h - H)) * d;
    float rms = 1.f;
    if (norm) {
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float x = rv_load(src + i);
            ss += x * x;
        }
        ss = rv_warp_sum(ss);
        rms = sqrtf(ss / (float)d + eps);
    }
    if (!norm && temp == 1.f && dst == src) return;
    for (int i = lane; i < d; i += 32) rv_store(dst + i, rv_load(src + i) / rms * temp);
}

// The same for key = value sizes of 8, 16, ..., 256: a lane owns 8 consecutive dimensions (one
// or two 16-byte accesses), d / 8 lanes cover a head and a warp covers 32 / (d / 8) heads.
__device__ __forceinline__ void qu_load8(const float* p, float (&v)[8]) {
    const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void qu_load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *(const uint4*)p;
    const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void qu_store8(float* p, const float (&v)[8]) {
    *(float4*)p = make_float4(v[0], v[1], v[2], v[3]);
    *(float4*)(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void qu_store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = (__nv_bfloat162*)&raw;
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *(uint4*)p = raw;
}

template <typename T>
__global__ void qk_unit_write_vec_kernel(T* __restrict__ rows, int row_stride, int n_tokens, int H,
                                         int G, int d, int norm, float eps, float coef, int every,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ slot_mapping,
                                         T* __restrict__ k_cache, T* __restrict__ v_cache) {
    rv_pdl_launch_dependents();
    const int lph = d >> 3, hpw = 32 / lph;                   // lanes per head, heads per warp
    const int heads_total = H + 2 * G;
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long item = warp * hpw + lane / lph;
    const int sub = lane % lph;
    const bool live = item < (long long)n_tokens * heads_total;
    int t = 0, h = 0, slot = 0;
    float temp = 1.f;
    if (live) {
        t = (int)(item / heads_total);
        h = (int)(item - (long long)t * heads_total);
        if (h >= H) slot = slot_mapping[t];
        if (h < H && every > 0) temp = 1.f + coef * logf((float)((positions[t] + 1) / every + 1));
    }
    rv_pdl_wait();
    const bool act = live && slot >= 0;
    T* src = rows + (size_t)t * row_stride + (size_t)h * d + sub * 8;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (act) qu_load8(src, v);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!act) return;
    if (h >= H + G) {                                          // a value head: copy
        qu_store8(v_cache + ((size_t)slot * G + (h - H - G)) * d + sub * 8, v);
        return;
    }
    T* dst = h < H ? src : k_cache + ((size_t)slot * G + (h - H)) * d + sub * 8;
    if (!norm && temp == 1.f && dst == src) return;
    const float rms = norm ? sqrtf(ss / (float)d + eps) : 1.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = v[i] / rms * temp;
    qu_store8(dst, v);
}

extern "C" int rv_qk_unit_write(void* rows, int dtype, int row_stride, int n_tokens, int H, int G,
                                int d, int dv, int norm, float eps, float coef, int every,
                                const int* positions, const int* slot_mapping, void* k_cache,
                                void* v_cache, void* stream) {
    if (n_tokens == 0) return 0;
    if (n_tokens < 0 || H <= 0 || G < 0 || d <= 0 || dv <= 0) RV_FAIL("qk_unit_write: bad sizes");
    if (every < 0 || (every > 0 && !positions))
        RV_FAIL("qk_unit_write: a query temperature needs positions and a step of at least 1");
    if (G > 0 && (!k_cache || !v_cache || !slot_mapping))
        RV_FAIL("qk_unit_write: key/value heads given without a cache to write");
    if (row_stride < H * d + G * (d + dv)) RV_FAIL("qk_unit_write: rows are too short");
    if (!norm && every == 0 && G == 0) return 0;
    const bool pow2 = d >= 8 && d <= 256 && (d & (d - 1)) == 0;
    if (pow2 && (G == 0 || d == dv) && row_stride % 8 == 0 && ((uintptr_t)rows & 15) == 0 &&
        ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0) {
        const int hpw = 32 / (d / 8);
        const long long vwarps = ((long long)n_tokens * (H + 2 * G) + hpw - 1) / hpw;
        const long long vblocks = (vwarps + 3) / 4;
        if (vblocks > 0x7fffffffLL) RV_FAIL("qk_unit_write: too many rows");
        RV_DISPATCH_DTYPE(dtype, "qk_unit_write",
                          (rv_launch(qk_unit_write_vec_kernel<T>, dim3((int)vblocks), dim3(128), 0,
                                     (cudaStream_t)stream, (T*)rows, row_stride, n_tokens, H, G, d,
                                     norm, eps, coef, every, positions, slot_mapping, (T*)k_cache,
                                     (T*)v_cache)));
        RV_CHECK_LAUNCH("qk_unit_write");
        return 0;
    }
    const long long warps = (long long)n_tokens * (H + 2 * G);
    const long long blocks = (warps + 3) / 4;
    if (blocks > 0x7fffffffLL) RV_FAIL("qk_unit_write: too many rows");
    RV_DISPATCH_DTYPE(dtype, "qk_unit_write",
                      (rv_launch(qk_unit_write_kernel<T>, dim3((int)blocks), dim3(128), 0,
                                 (cudaStream_t)stream, (T*)rows, row_stride, n_tokens, H, G, d, dv,
                                 norm, eps, coef, every, positions, slot_mapping, (T*)k_cache,
                                 (T*)v_cache)));
    RV_CHECK_LAUNCH("qk_unit_write");
    return 0;
}
