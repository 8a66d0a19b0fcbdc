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
