// minGRU scan over any mixture of prompt portions and single tokens.
//   rows  [N, 3 W] float32: the z | x | g product of each token (biases bz, bx not yet added)
//   z = sigmoid(rows_z + bz);  u = rows_x + bx;  c = u >= 0 ? u + 1/2 : sigmoid(u)
//   S_t = (1 - z_t) S_(t-1) + z_t c_t;  out_t = S_t * silu(rows_g)
// The state S is one float32 record [W] per request slot; it is read before a request's first
// token of the step and written after its last.  Everything is float32; out is the compute type.
//
// Two kernels.  "serial": one thread per (request, channel) walks the request's tokens; loads of
// neighbouring channels coalesce.  "chunked" (portions of RV_MINGRU_CHUNKED_FROM tokens or more):
// the recurrence S_t = a_t S_(t-1) + b_t is linear, so a block of (chunks x channels) threads lets
// every thread reduce its chunk of LEN tokens to (A, B) with S_end = A S_begin + B, walks the
// chunks' (A, B) in order through shared memory to get each chunk's S_begin, and then runs its
// chunk again from S_begin (chunks of up to 16 tokens keep their gates in registers instead of
// forming them twice).  Within one step the association of the sums differs from the serial
// order only by float32 rounding.
// Plain reference: tests/plain_ops.py mingru_scan.
#include "common.cuh"

#define RV_MINGRU_CHUNKED_FROM 64
#define RV_MINGRU_KEEP 16          // chunks up to this many tokens keep their gates in registers

// 1 / (1 + e^-x); the reciprocal is the correctly rounded one, as the division would give
__device__ __forceinline__ float rv_sigmoid(float x) { return __frcp_rn(1.f + expf(-x)); }

__device__ __forceinline__ void mingru_gate(float pz, float px, float bz, float bx, float& a,
                                            float& b) {
    const float z = rv_sigmoid(pz + bz);
    const float u = px + bx;
    const float c = u >= 0.f ? u + 0.5f : rv_sigmoid(u);
    a = 1.f - z;
    b = z * c;
}

template <typename TO>
__global__ void mingru_serial_kernel(const float* __restrict__ rows, const float* __restrict__ bias,
                                     float* __restrict__ state, const int* __restrict__ q_start,
                                     const int* __restrict__ state_slot, TO* __restrict__ out,
                                     int width, int min_len, int max_len) {
    rv_pdl_launch_dependents();
    const int r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int slot = state_slot[r];
    const int t0 = q_start[r], t1 = q_start[r + 1];
    if (slot < 0 || c >= width || t1 - t0 < min_len || t1 - t0 > max_len) return;
    const float bz = bias[c], bx = bias[width + c];
    rv_pdl_wait();
    float s = state[(size_t)slot * width + c];
    for (int t = t0; t < t1; ++t) {
        const float* row = rows + (size_t)t * 3 * width;
        float a, b;
        mingru_gate(row[c], row[width + c], bz, bx, a, b);
        s = a * s + b;
        const float g = row[2 * width + c];
        rv_store(out + (size_t)t * width + c, s * (g * rv_sigmoid(g)));
    }
    state[(size_t)slot * width + c] = s;
}

// blockDim = (CH channels, NC chunks); a request's portion is cut into NC chunks of
// len = ceil(T / NC) tokens.
template <typename TO, int CH, int NC>
__global__ void __launch_bounds__(CH * NC) mingru_chunked_kernel(const float* __restrict__ rows, const float* __restrict__ bias,
                                      float* __restrict__ state, const int* __restrict__ q_start,
                                      const int* __restrict__ state_slot, TO* __restrict__ out,
                                      int width, int min_len) {
    rv_pdl_launch_dependents();
    __shared__ float sa[NC][CH], sb[NC][CH];
    const int r = blockIdx.y;
    const int c = blockIdx.x * CH + threadIdx.x;
    const int k = threadIdx.y;
    const int slot = state_slot[r];
    const int t0 = q_start[r], t1 = q_start[r + 1];
    if (slot < 0 || t1 - t0 < min_len) return;          // the whole block leaves together
    const bool live = c < width;
    const float bz = live ? bias[c] : 0.f, bx = live ? bias[width + c] : 0.f;
    rv_pdl_wait();
    const int len = (t1 - t0 + NC - 1) / NC;
    const int b0 = min(t0 + k * len, t1), b1 = min(b0 + len, t1);
    float A = 1.f, B = 0.f;
    if (len <= RV_MINGRU_KEEP) {
        // short chunks: the gates of the first pass stay in registers for the second
        float ka[RV_MINGRU_KEEP], kb[RV_MINGRU_KEEP];
        // every load of the chunk is requested before any gate is formed
#pragma unroll
        for (int i = 0; i < RV_MINGRU_KEEP; ++i) {
            ka[i] = 0.f;
            kb[i] = 0.f;
            if (live && b0 + i < b1) {
                const float* row = rows + (size_t)(b0 + i) * 3 * width;
                ka[i] = row[c];
                kb[i] = row[width + c];
            }
        }
#pragma unroll
        for (int i = 0; i < RV_MINGRU_KEEP; ++i) {
            if (live && b0 + i < b1) {
                mingru_gate(ka[i], kb[i], bz, bx, ka[i], kb[i]);
                A *= ka[i];
                B = ka[i] * B + kb[i];
            } else {
                ka[i] = 1.f;
                kb[i] = 0.f;
            }
        }
        sa[k][threadIdx.x] = A;
        sb[k][threadIdx.x] = B;
        // the gate rows of the second pass travel while the chunks' (A, B) are walked
        float gv[RV_MINGRU_KEEP / 2];
#pragma unroll
        for (int i = 0; i < RV_MINGRU_KEEP / 2; ++i)
            gv[i] = (live && b0 + i < b1) ? rows[(size_t)(b0 + i) * 3 * width + 2 * width + c] : 0.f;
        __syncthreads();
        float s = live ? state[(size_t)slot * width + c] : 0.f;
        for (int j = 0; j < k; ++j) s = sa[j][threadIdx.x] * s + sb[j][threadIdx.x];
        if (!live) return;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            if (half == 1) {
#pragma unroll
                for (int i = 0; i < RV_MINGRU_KEEP / 2; ++i) {
                    const int t = b0 + RV_MINGRU_KEEP / 2 + i;
                    gv[i] = t < b1 ? rows[(size_t)t * 3 * width + 2 * width + c] : 0.f;
                }
            }
#pragma unroll
            for (int i = 0; i < RV_MINGRU_KEEP / 2; ++i) {
                const int ii = half * (RV_MINGRU_KEEP / 2) + i;
                if (b0 + ii < b1) {
                    s = ka[ii] * s + kb[ii];
                    rv_store(out + (size_t)(b0 + ii) * width + c, s * (gv[i] * rv_sigmoid(gv[i])));
                }
            }
        }
        if (k == NC - 1) state[(size_t)slot * width + c] = s;
        return;
    }
    if (live)
        for (int t = b0; t < b1; ++t) {
            const float* row = rows + (size_t)t * 3 * width;
            float a, b;
            mingru_gate(row[c], row[width + c], bz, bx, a, b);
            A *= a;
            B = a * B + b;
        }
    sa[k][threadIdx.x] = A;
    sb[k][threadIdx.x] = B;
    __syncthreads();
    float s = live ? state[(size_t)slot * width + c] : 0.f;
    for (int j = 0; j < k; ++j) s = sa[j][threadIdx.x] * s + sb[j][threadIdx.x];
    if (!live) return;
    for (int t = b0; t < b1; ++t) {
        const float* row = rows + (size_t)t * 3 * width;
        float a, b;
        mingru_gate(row[c], row[width + c], bz, bx, a, b);
        s = a * s + b;
        const float g = row[2 * width + c];
        rv_store(out + (size_t)t * width + c, s * (g * rv_sigmoid(g)));
    }
    if (k == NC - 1) state[(size_t)slot * width + c] = s;
}


extern "C" int rv_mingru_scan(const float* rows, const float* bias, float* state,
                              const int* q_start, const int* state_slot, void* out, int out_dtype,
                              int n_reqs, int max_q_len, int width, void* stream) {
    if (n_reqs == 0) return 0;
    if (n_reqs < 0 || width <= 0 || !state) RV_FAIL("mingru_scan: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    const bool chunked = max_q_len >= RV_MINGRU_CHUNKED_FROM;
    // requests of a step are served by one of the two kernels according to their own length,
    // whatever else is in the batch
    RV_DISPATCH_DTYPE(out_dtype, "mingru_scan", {
        rv_launch(mingru_serial_kernel<T>, dim3((width + 127) / 128, n_reqs), dim3(128), 0, s, rows,
                  bias, state, q_start, state_slot, (T*)out, width, 0,
                  chunked ? RV_MINGRU_CHUNKED_FROM - 1 : 0x7fffffff);
        // narrower channel tiles for narrower models, so that one long prompt still fills the
        // GPU (the tile follows from the width alone, never from what else is in the batch)
        if (chunked && width >= 4096)
            rv_launch(mingru_chunked_kernel<T, 32, 32>, dim3((width + 31) / 32, n_reqs), dim3(32, 32),
                      0, s, rows, bias, state, q_start, state_slot, (T*)out, width,
                      RV_MINGRU_CHUNKED_FROM);
        else if (chunked)
            rv_launch(mingru_chunked_kernel<T, 8, 128>, dim3((width + 7) / 8, n_reqs), dim3(8, 128),
                      0, s, rows, bias, state, q_start, state_slot, (T*)out, width,
                      RV_MINGRU_CHUNKED_FROM);
    });
    RV_CHECK_LAUNCH("mingru_scan");
    return 0;
}
