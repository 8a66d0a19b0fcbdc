// Layer norm with weight and bias, alone or fused with the addition into the float32 residual
// stream, and with a second layer norm applied to the rows that are being added:
//   d   = delta                         or  LN(delta; dw, db, deps)   (a norm after a sub-layer)
//   x   = resid + d  (written back to the stream unless `rows` selects rows)
//   out = LN(x; w, b, eps)
//   LN(v; w, b, e) = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + e) * w + b
// Without a stream (`resid` null) the rows of `delta` alone are normalised (w, b, eps).
// All statistics and sums are float32; the variance is taken from the deviations, in a second
// pass over the row, which is kept on chip.  One block per row.
// Plain reference: tests/plain_ops.py add_layernorm.
#include "common.cuh"

__device__ __forceinline__ float4 ln_load4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 ln_load4(const __nv_bfloat16* p) {
    const uint2 raw = *(const uint2*)p;
    const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x);
    const float2 b = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void ln_store4(float* p, float4 v) { *(float4*)p = v; }
__device__ __forceinline__ void ln_store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *(const unsigned*)&a;
    raw.y = *(const unsigned*)&b;
    *(uint2*)p = raw;
}

// mean and standard deviation (with eps inside the root) of a row whose values the block's
// threads hold in registers, CHUNKS groups of four each (group c of a thread is live when
// threadIdx.x + c * blockDim.x < nvec)
template <int CHUNKS>
__device__ __forceinline__ void ln_stats(const float (&v)[4 * CHUNKS], int nvec, int hidden,
                                         float eps, float* scratch, float& mean, float& sd) {
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
        if (threadIdx.x + c * blockDim.x < nvec) s += (v[4 * c] + v[4 * c + 1]) + (v[4 * c + 2] + v[4 * c + 3]);
    mean = rv_block_sum(s, scratch) / (float)hidden;
    float q = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
        if (threadIdx.x + c * blockDim.x < nvec) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float d = v[4 * c + k] - mean;
                q += d * d;
            }
        }
    sd = sqrtf(rv_block_sum(q, scratch) / (float)hidden + eps);
}

// General widths: the row lives in shared memory, every thread owns the elements
// threadIdx.x, threadIdx.x + blockDim.x, ...
template <typename TD, typename TO>
__global__ void add_layernorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                     const float* __restrict__ dw, const float* __restrict__ db,
                                     float deps, const float* __restrict__ w,
                                     const float* __restrict__ b, TO* __restrict__ out,
                                     const int* __restrict__ rows, int hidden, float eps) {
    rv_pdl_prologue();
    extern __shared__ float row[];
    __shared__ float scratch[33];
    const int m = blockIdx.x;
    const size_t in = (size_t)(rows ? rows[m] : m) * hidden;
    if (delta) {
        float s = 0.f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = rv_load(delta + in + i);
            row[i] = v;
            s += v;
        }
        if (dw) {
            const float mean = rv_block_sum(s, scratch) / (float)hidden;
            float q = 0.f;
            for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
                const float d = row[i] - mean;
                q += d * d;
            }
            const float sd = sqrtf(rv_block_sum(q, scratch) / (float)hidden + deps);
            for (int i = threadIdx.x; i < hidden; i += blockDim.x)
                row[i] = (row[i] - mean) / sd * dw[i] + db[i];
        }
    }
    float s = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float x = resid ? resid[in + i] : 0.f;
        if (delta) x += row[i];
        if (resid && delta && !rows) resid[in + i] = x;
        row[i] = x;
        s += x;
    }
    const float mean = rv_block_sum(s, scratch) / (float)hidden;
    float q = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row[i] - mean;
        q += d * d;
    }
    const float sd = sqrtf(rv_block_sum(q, scratch) / (float)hidden + eps);
    TO* o = out + (size_t)m * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        rv_store(o + i, (row[i] - mean) / sd * w[i] + b[i]);
}

// Widths that are multiples of 4 up to 8192: a thread keeps CHUNKS groups of four values in
// registers, every global value is loaded once with a 16-byte (float32) or
// 8-byte (bfloat16) access, and all loads of a stage are in flight together.
template <typename TD, typename TO, int CHUNKS>
__global__ void add_layernorm_vec_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                         const float* __restrict__ dw, const float* __restrict__ db,
                                         float deps, const float* __restrict__ w,
                                         const float* __restrict__ b, TO* __restrict__ out,
                                         const int* __restrict__ rows, int hidden, float eps) {
    rv_pdl_launch_dependents();
    __shared__ float scratch[33];
    const int m = blockIdx.x;
    const int nvec = hidden >> 2;
    // weights do not depend on the previous kernel: they are requested before the wait for it
    float4 wv[CHUNKS], bv[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec) {
            wv[c] = ln_load4(w + 4 * i);
            bv[c] = ln_load4(b + 4 * i);
        }
    }
    const int src = rows ? rows[m] : m;
    rv_pdl_wait();
    const size_t in = (size_t)src * hidden;
    float v[4 * CHUNKS];
    if (delta) {
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int i = threadIdx.x + c * blockDim.x;
            if (i < nvec) {
                const float4 d = ln_load4(delta + in + 4 * i);
                v[4 * c] = d.x; v[4 * c + 1] = d.y; v[4 * c + 2] = d.z; v[4 * c + 3] = d.w;
            }
        }
        if (dw) {
            float mean, sd;
            ln_stats<CHUNKS>(v, nvec, hidden, deps, scratch, mean, sd);
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                const int i = threadIdx.x + c * blockDim.x;
                if (i < nvec) {
                    const float4 a = ln_load4(dw + 4 * i), o = ln_load4(db + 4 * i);
                    v[4 * c] = (v[4 * c] - mean) / sd * a.x + o.x;
                    v[4 * c + 1] = (v[4 * c + 1] - mean) / sd * a.y + o.y;
                    v[4 * c + 2] = (v[4 * c + 2] - mean) / sd * a.z + o.z;
                    v[4 * c + 3] = (v[4 * c + 3] - mean) / sd * a.w + o.w;
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec) {
            float4 x = resid ? ln_load4(resid + in + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (delta) {
                x.x += v[4 * c]; x.y += v[4 * c + 1]; x.z += v[4 * c + 2]; x.w += v[4 * c + 3];
                if (resid && !rows) ln_store4(resid + in + 4 * i, x);
            }
            v[4 * c] = x.x; v[4 * c + 1] = x.y; v[4 * c + 2] = x.z; v[4 * c + 3] = x.w;
        }
    }
    float mean, sd;
    ln_stats<CHUNKS>(v, nvec, hidden, eps, scratch, mean, sd);
    TO* o = out + (size_t)m * hidden;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec)
            ln_store4(o + 4 * i, make_float4((v[4 * c] - mean) / sd * wv[c].x + bv[c].x,
                                             (v[4 * c + 1] - mean) / sd * wv[c].y + bv[c].y,
                                             (v[4 * c + 2] - mean) / sd * wv[c].z + bv[c].z,
                                             (v[4 * c + 3] - mean) / sd * wv[c].w + bv[c].w));
    }
}

template <typename TD, typename TO>
static int add_layernorm_launch(float* resid, const void* delta, const float* dw, const float* db,
                                float deps, const float* w, const float* b, void* out,
                                const int* rows, int n_rows, int hidden, float eps,
                                cudaStream_t stream) {
    const bool aligned = ((uintptr_t)resid % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                         ((uintptr_t)b % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
                         (!delta || (uintptr_t)delta % 16 == 0) &&
                         (!dw || ((uintptr_t)dw % 16 == 0 && (uintptr_t)db % 16 == 0));
    if (hidden % 4 == 0 && hidden <= 8192 && aligned) {
        const int nvec = hidden / 4;
        int chunks = 1;
        while ((nvec + chunks - 1) / chunks > 512) chunks *= 2;          // at most 4
        const int threads = (((nvec + chunks - 1) / chunks + 31) / 32) * 32;
#define RV_LN_VEC(C)                                                                           \
    rv_launch(add_layernorm_vec_kernel<TD, TO, C>, dim3(n_rows), dim3(threads), 0, stream, resid, \
              (const TD*)delta, dw, db, deps, w, b, (TO*)out, rows, hidden, eps)
        if (chunks == 1) RV_LN_VEC(1);
        else if (chunks == 2) RV_LN_VEC(2);
        else RV_LN_VEC(4);
#undef RV_LN_VEC
        RV_CHECK_LAUNCH("add_layernorm");
        return 0;
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) RV_FAIL("add_layernorm: width %d exceeds the shared-memory row", hidden);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(add_layernorm_kernel<TD, TO>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RV_FAIL("add_layernorm: %s", cudaGetErrorString(e));
    }
    rv_launch(add_layernorm_kernel<TD, TO>, dim3(n_rows), dim3(hidden >= 1024 ? 256 : 128), smem,
              stream, resid, (const TD*)delta, dw, db, deps, w, b, (TO*)out, rows, hidden, eps);
    RV_CHECK_LAUNCH("add_layernorm");
    return 0;
}

extern "C" int rv_add_layernorm(float* resid, const void* delta, int delta_dtype, const float* dw,
                                const float* db, float deps, const float* w, const float* b,
                                void* out, int out_dtype, const int* rows, int n_rows, int hidden,
                                float eps, void* stream) {
    if (n_rows == 0) return 0;
    if (n_rows < 0 || hidden <= 0) RV_FAIL("add_layernorm: bad sizes");
    if (!resid && !delta) RV_FAIL("add_layernorm: neither a stream nor rows to normalise");
    if (!resid && (rows || dw)) RV_FAIL("add_layernorm: without a stream it takes plain rows, all of them");
    if ((dw == nullptr) != (db == nullptr) || (dw && !delta))
        RV_FAIL("add_layernorm: incomplete arguments for the norm of the added rows");
    cudaStream_t s = (cudaStream_t)stream;
#define RV_LN(TD, TO) \
    return add_layernorm_launch<TD, TO>(resid, delta, dw, db, deps, w, b, out, rows, n_rows, hidden, eps, s)
    if (delta_dtype == RV_DTYPE_F32 && out_dtype == RV_DTYPE_F32) RV_LN(float, float);
    if (delta_dtype == RV_DTYPE_BF16 && out_dtype == RV_DTYPE_BF16) RV_LN(__nv_bfloat16, __nv_bfloat16);
    if (delta_dtype == RV_DTYPE_F32 && out_dtype == RV_DTYPE_BF16) RV_LN(float, __nv_bfloat16);
    if (delta_dtype == RV_DTYPE_BF16 && out_dtype == RV_DTYPE_F32) RV_LN(__nv_bfloat16, float);
#undef RV_LN
    RV_FAIL("add_layernorm: unknown dtype codes %d, %d", delta_dtype, out_dtype);
}
