// Rotation of the first `rot_dims` dimensions of every query and key head and the write of keys
// and values into the paged cache, for rows laid out as
//   [ q: H heads of d | k: G heads of d | v: G heads of dv | anything else ]
// (G = 0: the rows carry queries only and no cache is written).  Dimension i < rot_dims/2 of a
// head turns with dimension i + rot_dims/2 by the angle position * freq[i]; angle, sine and
// cosine are float32 and are formed here, so no table over positions exists.  Queries are
// rotated in place, keys go rotated to the key pages, values as they are to the value pages.
// One warp per (token, head).  Plain reference: tests/plain_ops.py rope_partial_write.
#include "common.cuh"

template <typename T>
__global__ void rope_partial_write_kernel(T* __restrict__ rows, int row_stride, int n_tokens, int H,
                                          int G, int d, int dv, const float* __restrict__ freq,
                                          int rot_dims, const int* __restrict__ positions,
                                          const int* __restrict__ slot_mapping,
                                          T* __restrict__ k_cache, T* __restrict__ v_cache) {
    rv_pdl_launch_dependents();
    const int heads_total = H + 2 * G;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= (long long)n_tokens * heads_total) return;
    const int t = (int)(warp / heads_total);
    const int h = (int)(warp - (long long)t * heads_total);
    const int half = rot_dims >> 1;
    const int slot = h >= H ? slot_mapping[t] : 0;
    const float pos = (freq && h < H + G) ? (float)positions[t] : 0.f;
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
    if (freq)
        for (int i = lane; i < half; i += 32) {
            const float u = rv_load(src + i), v = rv_load(src + i + half);
            float sn, cs;
            sincosf(pos * freq[i], &sn, &cs);
            rv_store(dst + i, u * cs - v * sn);
            rv_store(dst + i + half, v * cs + u * sn);
        }
    if (dst != src)
        for (int i = (freq ? rot_dims : 0) + lane; i < d; i += 32) dst[i] = src[i];
}

extern "C" int rv_rope_partial_write(void* rows, int dtype, int row_stride, int n_tokens, int H,
                                     int G, int d, int dv, const float* freq, int rot_dims,
                                     const int* positions, const int* slot_mapping, void* k_cache,
                                     void* v_cache, void* stream) {
    if (n_tokens == 0) return 0;
    if (n_tokens < 0 || H <= 0 || G < 0 || d <= 0 || dv <= 0) RV_FAIL("rope_partial_write: bad sizes");
    if (freq && (rot_dims % 2 || rot_dims > d || rot_dims < 0 || !positions))
        RV_FAIL("rope_partial_write: %d turning dimensions do not fit a head of %d", rot_dims, d);
    if (G > 0 && (!k_cache || !v_cache || !slot_mapping))
        RV_FAIL("rope_partial_write: key/value heads given without a cache to write");
    if (row_stride < H * d + G * (d + dv)) RV_FAIL("rope_partial_write: rows are too short");
    if (!freq && G == 0) return 0;
    const long long warps = (long long)n_tokens * (H + 2 * G);
    const long long blocks = (warps + 3) / 4;
    if (blocks > 0x7fffffffLL) RV_FAIL("rope_partial_write: too many rows");
    RV_DISPATCH_DTYPE(dtype, "rope_partial_write",
                      (rv_launch(rope_partial_write_kernel<T>, dim3((int)blocks), dim3(128), 0,
                                 (cudaStream_t)stream, (T*)rows, row_stride, n_tokens, H, G, d, dv,
                                 freq, rot_dims, positions, slot_mapping, (T*)k_cache, (T*)v_cache)));
    RV_CHECK_LAUNCH("rope_partial_write");
    return 0;
}
